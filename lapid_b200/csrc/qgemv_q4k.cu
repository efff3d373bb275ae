// Q4_K, Q5_K and Q6_K decode GEMV, fast path for 1..8 activation rows (arithmetic: see qgemv.cu; this file only
// changes how the work is laid out on the machine).
//
//  * Weights reach the SM through per-warp rings of shared-memory stages filled by the bulk-copy
//    engine (`cp.async.bulk` global -> shared, completion on an mbarrier): one instruction, issued
//    by one lane, moves the 4.6 KB of contiguous weight bytes a warp consumes per step (32
//    super-blocks). No registers or load/store-unit slots are spent on the stream, requests are
//    whole 128-byte lines, and a warp never waits for another warp.
//  * One lane owns one 144-byte super-block of the stage (nine conflict-free 128-bit shared
//    loads: the lane stride of 144 = 9*16 bytes walks all bank groups). G lanes (8, 16 or 32,
//    the power of two covering K/256) share one weight row; a warp works on 32/G rows at once
//    and finishes a row with log2(G) shuffles.
//  * The 12 packed scale/min bytes of a block are decoded for all eight sub-blocks with eight
//    logic operations on three words; high nibbles are used in place (16*q, an exact power of
//    two folded into the scale), so unpacking costs two logic operations per word.
//  * The int8 activations live in shared memory as one 336-byte record per (row, super-block):
//    four times [64 quants | da_2p da_2p+1 bs_2p bs_2p+1], padded so that the lanes' 128-bit
//    reads (stride 336 = 21*16 bytes) are bank-conflict free. The pre-pass kernel writes the
//    records in this layout; the prologue copies them with `cp.async`, all copies in flight at
//    once (one L2 round trip, hidden behind the weight requests).
//  * The rings are filled before the programmatic-dependent-launch wait: weights never depend on
//    the kernel that produces the activations, so they stream while that kernel still runs.
//  * Every mbarrier wait is bounded; a wait that gives up records it in a host-visible status
//    word and the kernel runs to its end (with a wrong result that the host then rejects).
#include "common.cuh"
#include "kernels.h"
#include "tp_ll.cuh"

namespace lb {

template <int FMT> struct Blk {
    static constexpr int BYTES = FMT == FMT_Q4K ? Q4K_BYTES : FMT == FMT_Q5K ? Q5K_BYTES : Q6K_BYTES;
    // 32 blocks by one bulk copy. Q4_K: 4608 bytes, always 16-byte aligned. Q6_K: 6720 bytes that may
    // start anywhere on a 2-byte boundary: the copy starts at the 16-byte boundary below and is up to
    // 16 bytes longer; the consumers add the same offset.
    static constexpr int STAGE = FMT == FMT_Q6K ? 32 * BYTES + 16 : 32 * BYTES;  // (Q5_K: 176 = 11 * 16 bytes, aligned like Q4_K)
};
constexpr int BAR_BYTES = 256;  // warps * STAGES * 8 <= 256
// room behind the activation records for results parked in early mode: 4 warps * (16 / M) tasks * up to 4 rows * M floats
__host__ __device__ constexpr size_t pend_bytes(int rows) { return rows <= 2 ? (size_t)4 * 16 * 4 * 4 : 0; }

__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(s32(dst)),
                 "l"(src), "r"(bytes), "r"(s32(bar))
                 : "memory");
}
// Bounded wait for the phase with the given parity. Returns false when it gave up.
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

// unsigned bytes of a (0..240) times signed bytes of b
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ float u8f(uint32_t w, int byte) { return (float)((w >> (8 * byte)) & 0xffu); }

// float(byte `sel` of w) * d, exactly: the byte is planted in the mantissa of 2^23 with one PRMT and
// the bias is removed inside one fused multiply-add (d * (2^23 + b) - d * 2^23 = d * b needs 17
// bits, so the result is exact and equals the reference's separately rounded d * f32(b)).
__device__ __forceinline__ float scale_byte(uint32_t w, uint32_t sel, float d, float neg_d23) {
    return fmaf(d, __uint_as_float(__byte_perm(w, 0x4B000000u, sel)), neg_d23);
}

// One 64-weight pair of a super-block against one activation row: two groups of 32.
__device__ __forceinline__ float pair_dot(const uint32_t (&v)[8], const uint32_t (&al)[8], const uint32_t (&ah)[8], float s0,
                                          float m0, float s1, float m1, float da0, float da1, float bs0, float bs1,
                                          float acc) {
    int l0 = 0, l1 = 0, h0 = 0, h1 = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        l0 = dp4a_us(v[i] & 0x0F0F0F0Fu, al[i], l0);
        l1 = dp4a_us(v[i + 4] & 0x0F0F0F0Fu, al[i + 4], l1);
        h0 = dp4a_us(v[i] & 0xF0F0F0F0u, ah[i], h0);
        h1 = dp4a_us(v[i + 4] & 0xF0F0F0F0u, ah[i + 4], h1);
    }
    acc = fmaf(s0 * da0, (float)(l0 + l1), acc);
    acc = fmaf(-m0, bs0, acc);
    acc = fmaf(s1 * da1, (float)(h0 + h1), acc);
    acc = fmaf(-m1, bs1, acc);
    return acc;
}

// The same for Q5_K: 5-bit weights, already unpacked to bytes 0..31 (lo: sub-block 2p, hi: sub-block 2p + 1).
__device__ __forceinline__ float pair_dot5(const uint32_t (&lo)[8], const uint32_t (&hi)[8], const uint32_t (&al)[8],
                                           const uint32_t (&ah)[8], float s0, float m0, float s1, float m1, float da0, float da1,
                                           float bs0, float bs1, float acc) {
    int l0 = 0, l1 = 0, h0 = 0, h1 = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        l0 = dp4a_us(lo[i], al[i], l0);
        l1 = dp4a_us(lo[i + 4], al[i + 4], l1);
        h0 = dp4a_us(hi[i], ah[i], h0);
        h1 = dp4a_us(hi[i + 4], ah[i + 4], h1);
    }
    acc = fmaf(s0 * da0, (float)(l0 + l1), acc);
    acc = fmaf(-m0, bs0, acc);
    acc = fmaf(s1 * da1, (float)(h0 + h1), acc);
    acc = fmaf(-m1, bs1, acc);
    return acc;
}

// `n` words starting at a 2-byte aligned shared address (Q6_K blocks are 210 bytes long, so every
// other block of a stage starts in the middle of a word): aligned loads plus a funnel shift.
template <int N> __device__ __forceinline__ void lds_words_align2(const uint8_t *p, uint32_t (&w)[N]) {
    const uint32_t *q = (const uint32_t *)((uintptr_t)p & ~(uintptr_t)3);
    const uint32_t sh = ((uint32_t)(uintptr_t)p & 2u) * 8u;
    uint32_t prev = q[0];
#pragma unroll
    for (int i = 0; i < N; i++) {
        const uint32_t nxt = q[i + 1];
        w[i] = __funnelshift_r(prev, nxt, sh);
        prev = nxt;
    }
}

// One 32-element Q6_K sub-block pair member against one activation group: two 16-element halves
// with their own int8 scales, v = sc0*dot0 + sc1*dot1 (crates/lapid-cpu/src/kquant.rs:224-233).
__device__ __forceinline__ float q6_group(const uint32_t (&q)[8], const uint32_t (&a)[8], float sc0, float sc1) {
    int d0 = 0, d1 = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        d0 = __dp4a((int)q[i], (int)a[i], d0);
        d1 = __dp4a((int)q[i + 4], (int)a[i + 4], d1);
    }
    return fmaf(sc1, (float)d1, sc0 * (float)d0);
}

// Warps per CTA: small CTAs for one or two rows (many CTAs per SM, so that one slot can be left to
// the next kernel), larger ones beyond, where the activation records are the bigger share of the
// shared memory and are better amortised over more warps.
template <int M> struct Shape { static constexpr int WARPS = M <= 2 ? 4 : 8, MIN_CTAS = M <= 2 ? 5 : 2; };

// MOE (Kernel::MatMulId at decode sizes; M == 1, NG == 1): the weight operand is a stack of matrices and
// every (token, slot) pair is a one-row GEMV against the matrix its expert id selects. The pairs'
// tasks form one list (a task never straddles two pairs), the activation records of all tokens
// sit in shared memory and a task reads the records of its pair's token.
// EARLY (one or two rows; GemvArgs::early of every member): see below.
template <int FMT, int M, int G, int NG, bool MOE = false, bool EARLY = false>
__global__ void __launch_bounds__(Shape<M>::WARPS * 32, Shape<M>::MIN_CTAS) qgemv_kq_fast_kernel(GemvGroupT<NG> grp) {
    static_assert(!MOE || (M == 1 && NG == 1), "expert-indexed launches are one-row, one-item launches");
    static_assert(!EARLY || (M <= 2 && !MOE), "early mode is built for one and two rows");
    constexpr int STAGES = 2;
    constexpr int BB = Blk<FMT>::BYTES, STAGE_BYTES = Blk<FMT>::STAGE;
    constexpr int FAST_WARPS = Shape<M>::WARPS, FAST_THREADS = FAST_WARPS * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int RPW = 32 / G;
    constexpr bool DEFER = EARLY;  // park results instead of waiting at the first store
    constexpr int PEND_MAX = 16 / M;
    const int sub = lane / G, gl = lane % G;
    // A launch covers up to GEMV_GROUP_MAX independent projections with the same format, row count
    // and K (q/k/v, gate/up): their tasks (32/G weight rows each) form one list, so the weight
    // stream does not stop between them and small matrices share one launch.
    const uint32_t nblk = grp.item[0].k / QK;
    const uint32_t iters = (nblk + G - 1) / G;
    const uint32_t tasks = grp.task_end[grp.count - 1];
    const uint32_t tpp = MOE ? (grp.item[0].n + RPW - 1) / RPW : 0;  // tasks per (token, slot) pair
    // the matrix of a pair; an id outside the stack is reported and replaced by 0
    auto expert_matrix = [&](uint32_t pair) -> const uint8_t * {
        const int32_t id = grp.item[0].ids[pair];
        const bool bad = id < 0 || (uint32_t)id >= grp.item[0].id_e;
        if (bad && grp.item[0].status) atomicOr(grp.item[0].status, 128);
        return grp.item[0].w + (bad ? 0 : (uint64_t)id * grp.item[0].id_stride);
    };
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
    // CTA c owns tasks [t_lo, t_hi); its warps take them round-robin
    const uint32_t t_lo = (uint32_t)(((uint64_t)tasks * blockIdx.x) / gridDim.x);
    const uint32_t t_hi = (uint32_t)(((uint64_t)tasks * (blockIdx.x + 1)) / gridDim.x);

    uint64_t *bars = (uint64_t *)smem + warp * STAGES;
    uint8_t *ring = smem + BAR_BYTES + (size_t)warp * (STAGES * STAGE_BYTES);
    uint8_t *acts = smem + BAR_BYTES + (size_t)FAST_WARPS * STAGES * STAGE_BYTES;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) mbar_init(bars + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // producer cursor (task, step within the task, ring slot)
    uint32_t pt = t_lo + warp, pit = 0, pslot = 0;
    // One stage = the contiguous run of super-blocks the warp consumes in one step: all blocks of
    // its 32/G rows when a row fits in G lanes, else 32 blocks of its single row.
    auto issue = [&]() {
        if (pt >= t_hi) return;
        if (lane == 0) {
            uint32_t local;
            const int item = locate(pt, local);
            const uint32_t n = grp.item[item].n;
            const uint8_t *wbase = grp.item[item].w;
            if constexpr (MOE) {
                wbase = expert_matrix(local / tpp);
                local %= tpp;
            }
            const uint32_t row0 = local * RPW;
            uint32_t first, count;
            if (iters == 1) {
                first = row0 * nblk;
                count = min((uint32_t)RPW, n - row0) * nblk;
            } else {
                first = row0 * nblk + pit * 32;
                count = min(32u, nblk - pit * 32);
            }
            const uint8_t *src = wbase + (uint64_t)first * BB;
            const uint32_t skew = (uint32_t)((uintptr_t)src & 15u);  // 0 for Q4_K
            const uint32_t bytes = (skew + count * BB + 15u) & ~15u;
            mbar_expect_tx(bars + pslot, bytes);
            bulk_g2s(ring + (size_t)pslot * STAGE_BYTES, src - skew, bytes, bars + pslot);
        }
        pslot ^= 1;
        if (++pit == iters) {
            pit = 0;
            pt += FAST_WARPS;
        }
    };
    if constexpr (MOE) {  // the expert ids come from the kernel before this one: nothing can be fetched ahead of it
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    issue();
    issue();
    // early (GemvArgs::early): the activations are older than the kernel in front of this one, so they are
    // fetched, and the first results computed, while that kernel still runs; only the stores wait for it
    constexpr bool early = EARLY;
    auto copy_acts = [&]() {
        const uint32_t chunks = (MOE ? grp.item[0].rows : M) * nblk * (REC / 16);
        for (int i = 0; i < grp.count; i++) {
            if (!grp.act_copy[i]) continue;  // same activations as an earlier projection of the group
            const uint8_t *src = (const uint8_t *)grp.item[i].qa;
            uint8_t *dst = acts + grp.act_off[i];
            for (uint32_t c = threadIdx.x; c < chunks; c += FAST_THREADS)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s32(dst + 16 * c)), "l"(src + 16 * (size_t)c) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (early) copy_acts();
    if constexpr (!MOE) {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        if (!early) asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    bool waited = !early;

    __shared__ TpPushCtx tp_ctx;  // only the first member of a launch may push (tensor-parallel launches are never grouped)
    if (grp.item[0].tp && threadIdx.x == 0) tp_push_ctx_load(&tp_ctx, grp.item[0].tp);
    if (!early) copy_acts();
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    // results parked while the kernel in front still runs (early mode, one or two rows): [task][row of the task][M]
    float *pend = (float *)(acts + grp.act_bytes) + warp * (PEND_MAX * RPW * M);
    uint32_t npend = 0, pend_first = 0;
    auto flush_pending = [&]() {
        for (uint32_t q = 0; q < npend; q++) {
            uint32_t local;
            const int item = locate(pend_first + q * FAST_WARPS, local);
            const GemvArgs &p = grp.item[item];
            const uint32_t row = local * RPW + sub;
            if (gl == 0 && row < p.n) {
#pragma unroll
                for (int r = 0; r < M; r++) {
                    float v = pend[(q * RPW + sub) * M + r];
                    const uint32_t bt = r / p.m, i = r % p.m;
                    if (p.extra && !p.epi.n) v += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)i * p.ex_s1 + (int64_t)row * p.ex_s2];
                    p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)i * p.out_rs + row] = v;
                }
            }
        }
        npend = 0;
    };

    float acc[M];
    bool healthy = true;
    uint32_t cslot = 0, cpar = 0;
    for (uint32_t t = t_lo + warp; t < t_hi; t += FAST_WARPS) {
        uint32_t local;
        const int item = locate(t, local);
        const GemvArgs &p = grp.item[item];
        const uint32_t n = p.n;
        const uint8_t *iacts = acts + grp.act_off[item];
        const uint8_t *wbase = p.w;
        uint32_t pair = 0;
        if constexpr (MOE) {
            pair = local / tpp;
            local %= tpp;
            wbase = expert_matrix(pair);
            iacts += (size_t)(pair / p.id_r) * nblk * REC;  // the records of the pair's token
        }
        const uint32_t row = local * RPW + sub;
#pragma unroll
        for (int r = 0; r < M; r++) acc[r] = 0.0f;
        for (uint32_t it = 0; it < iters; it++) {
            if (healthy && !mbar_wait(bars + cslot, cpar)) {
                healthy = false;
                if (lane == 0 && grp.item[0].status) atomicOr(grp.item[0].status, 1);
            }
            const uint32_t b = it * G + gl;
            if (healthy && row < n && b < nblk && gl < nblk) {
                // the stage starts at the 16-byte boundary below its first block (Q6_K; see Blk)
                const uint32_t first_blk = iters == 1 ? local * RPW * nblk : local * RPW * nblk + it * 32;
                const uint32_t skew = FMT != FMT_Q6K ? 0u : (uint32_t)(((uintptr_t)wbase + (uint64_t)first_blk * BB) & 15u);
                const uint8_t *blk = ring + (size_t)cslot * STAGE_BYTES + skew + (size_t)(iters == 1 ? sub * nblk + gl : gl) * BB;
                if constexpr (FMT == FMT_Q4K || FMT == FMT_Q5K) {
                    const uint4 h = *(const uint4 *)blk;
                    const float d = half_bits_to_float(h.x & 0xffff), dmin = half_bits_to_float(h.x >> 16);
                    const float nd = d * -8388608.0f, ndmin = dmin * -8388608.0f;
                    const uint32_t w0 = h.y, w1 = h.z, w2 = h.w;
                    // bytes: sc_lo = scales 0..3, sc_hi = scales 4..7, likewise the mins
                    const uint32_t sc_lo = w0 & 0x3F3F3F3Fu, mn_lo = w1 & 0x3F3F3F3Fu;
                    const uint32_t sc_hi = (w2 & 0x0F0F0F0Fu) | (((w0 >> 6) & 0x03030303u) << 4);
                    const uint32_t mn_hi = ((w2 >> 4) & 0x0F0F0F0Fu) | (((w1 >> 6) & 0x03030303u) << 4);
#pragma unroll
                    for (int pp = 0; pp < 4; pp++) {
                        const uint32_t scw = pp < 2 ? sc_lo : sc_hi, mnw = pp < 2 ? mn_lo : mn_hi;
                        const uint32_t sel0 = 0x7440u + 2 * (pp & 1), sel1 = sel0 + 1;  // {byte, 0, 0, 0x4B}
                        const float s0 = scale_byte(scw, sel0, d, nd), m0 = scale_byte(mnw, sel0, dmin, ndmin);
                        // the high nibbles are used as 16*q: fold the exact factor 1/16 into their scale
                        constexpr int QS = FMT == FMT_Q5K ? 48 : 16;  // Q5_K: the fifth bits qh[32] sit between the header and the nibbles
                        const float s1 = scale_byte(scw, sel1, d, nd) * (FMT == FMT_Q5K ? 1.0f : 0.0625f), m1 = scale_byte(mnw, sel1, dmin, ndmin);
                        const uint4 qa_ = *(const uint4 *)(blk + QS + 32 * pp), qb_ = *(const uint4 *)(blk + QS + 16 + 32 * pp);
                        uint32_t v[8] = {qa_.x, qa_.y, qa_.z, qa_.w, qb_.x, qb_.y, qb_.z, qb_.w};
                        uint32_t vh[8];  // Q5_K: the high nibbles shifted down, with their fifth bits
                        if constexpr (FMT == FMT_Q5K) {
                            // bit s of qh[l] belongs to element 32 s + l: sub-blocks 2 pp (low nibbles) and 2 pp + 1
                            const uint4 ha_ = *(const uint4 *)(blk + 16), hb_ = *(const uint4 *)(blk + 32);
                            const uint32_t hq[8] = {ha_.x, ha_.y, ha_.z, ha_.w, hb_.x, hb_.y, hb_.z, hb_.w};
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                vh[i] = ((v[i] >> 4) & 0x0F0F0F0Fu) | (((hq[i] >> (2 * pp + 1)) & 0x01010101u) << 4);
                                v[i] = (v[i] & 0x0F0F0F0Fu) | (((hq[i] >> (2 * pp)) & 0x01010101u) << 4);
                            }
                        }
#pragma unroll
                        for (int r = 0; r < M; r++) {
                            const uint4 *rec = (const uint4 *)(iacts + ((size_t)r * nblk + b) * REC + 80 * pp);
                            const uint4 a0 = rec[0], a1 = rec[1], a2 = rec[2], a3 = rec[3], sc = rec[4];
                            const uint32_t al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                            const uint32_t ah[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
                            if constexpr (FMT == FMT_Q5K)
                                acc[r] = pair_dot5(v, vh, al, ah, s0, m0, s1, m1, __uint_as_float(sc.x), __uint_as_float(sc.y),
                                                   __uint_as_float(sc.z), __uint_as_float(sc.w), acc[r]);
                            else
                                acc[r] = pair_dot(v, al, ah, s0, m0, s1, m1, __uint_as_float(sc.x), __uint_as_float(sc.y),
                                                  __uint_as_float(sc.z), __uint_as_float(sc.w), acc[r]);
                        }
                    }
                } else {
                    // Q6_K: ql[128] | qh[64] | int8 sc[16] | f16 d; the block is only 2-byte aligned
                    const float d = half_bits_to_float((uint32_t)blk[208] | ((uint32_t)blk[209] << 8));
#pragma unroll
                    for (int nh = 0; nh < 2; nh++) {  // the two 128-element halves
                        uint32_t ql[16], qh[8], scw[2];
                        lds_words_align2<16>(blk + 64 * nh, ql);
                        lds_words_align2<8>(blk + 128 + 32 * nh, qh);
                        lds_words_align2<2>(blk + 192 + 8 * nh, scw);
#pragma unroll
                        for (int j = 0; j < 2; j++) {  // record pair 2*nh + j: sub-blocks w = 2j (ql bytes 0..31) and 2j+1 (32..63)
                            const int pp = 2 * nh + j;
                            uint32_t q0[8], q1[8];
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                const uint32_t lo0 = (ql[i] >> (4 * j)) & 0x0F0F0F0Fu, lo1 = (ql[8 + i] >> (4 * j)) & 0x0F0F0F0Fu;
                                const uint32_t hi0 = ((qh[i] >> (4 * j)) & 0x03030303u) << 4, hi1 = ((qh[i] >> (4 * j + 2)) & 0x03030303u) << 4;
                                q0[i] = __vsub4(lo0 | hi0, 0x20202020u);  // signed quants -32..31
                                q1[i] = __vsub4(lo1 | hi1, 0x20202020u);
                            }
                            const float s00 = (float)(int8_t)(scw[j] & 0xff), s01 = (float)(int8_t)((scw[j] >> 8) & 0xff);
                            const float s10 = (float)(int8_t)((scw[j] >> 16) & 0xff), s11 = (float)(int8_t)(scw[j] >> 24);
#pragma unroll
                            for (int r = 0; r < M; r++) {
                                const uint4 *rec = (const uint4 *)(iacts + ((size_t)r * nblk + b) * REC + 80 * pp);
                                const uint4 a0 = rec[0], a1 = rec[1], a2 = rec[2], a3 = rec[3], sc = rec[4];
                                const uint32_t al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                                const uint32_t ah[8] = {a2.x, a2.y, a2.z, a2.w, a3.x, a3.y, a3.z, a3.w};
                                float a_ = acc[r];
                                a_ = fmaf(d * __uint_as_float(sc.x), q6_group(q0, al, s00, s01), a_);
                                a_ = fmaf(d * __uint_as_float(sc.y), q6_group(q1, ah, s10, s11), a_);
                                acc[r] = a_;
                            }
                        }
                    }
                }
            }
            __syncwarp();  // every lane is done reading the slot before it is refilled
            issue();
            cslot ^= 1;
            if (cslot == 0) cpar ^= 1;
        }
        if (DEFER && !waited) {
            // early mode: the kernel in front still runs, so nothing may be written yet. Park the task's results
            // in shared memory and go on computing; the stores follow once that kernel has completed.
            if (npend == 0) pend_first = t;
#pragma unroll
            for (int r = 0; r < M; r++) {
                float v = acc[r];
#pragma unroll
                for (int o = G / 2; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (gl == 0) pend[(npend * RPW + sub) * M + r] = v;
            }
            if (++npend == PEND_MAX) {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                waited = true;
                flush_pending();
            }
            continue;
        }
        if (!waited) {  // nothing is written before the kernel in front has completed
            asm volatile("griddepcontrol.wait;" ::: "memory");
            waited = true;
        }
#pragma unroll
        for (int r = 0; r < M; r++) {
            float v = acc[r];
#pragma unroll
            for (int o = G / 2; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (gl == 0 && row < n) {
                const uint32_t bt = r / p.m, i = r % p.m;
                if (p.extra && !p.epi.n) v += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)i * p.ex_s1 + (int64_t)row * p.ex_s2];
                if constexpr (MOE) p.out[p.out_off + (uint64_t)pair * n + row] = v;
                else if (p.tp) tp_push_value(&tp_ctx, (uint64_t)r * n + row, v);  // row-parallel partial: to every rank
                else p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)i * p.out_rs + row] = v;
            }
        }
    }
    // a warp without a task still may not let its CTA (and with it the grid) end before the kernel in front
    // has: later kernels take this grid's completion as the completion of everything before it
    if (!waited) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if constexpr (DEFER) flush_pending();
    }
}

static int g_cta_cap = 0;  // 0 = as many CTAs per SM as fit; set through qgemv_q4k_fast_set_cta_cap

void qgemv_q4k_fast_set_cta_cap(int cap) { g_cta_cap = cap; }

template <int FMT, int M, int G, int NG, bool MOE = false, bool EARLY = false>
static cudaError_t launch_fast_n(GemvGroupT<NG> &g, int sm_count, bool pdl, cudaStream_t stream) {
    if constexpr (!EARLY && !MOE && M <= 2) {  // every member early, no tensor-parallel push: the early instantiation
        bool early = pdl;
        for (int i = 0; i < g.count; i++) early = early && g.item[i].early != 0 && g.item[i].tp == nullptr;
        if (early) return launch_fast_n<FMT, M, G, NG, MOE, true>(g, sm_count, pdl, stream);
    }
    auto kern = qgemv_kq_fast_kernel<FMT, M, G, NG, MOE, EARLY>;
    constexpr int FAST_WARPS = Shape<M>::WARPS, FAST_THREADS = FAST_WARPS * 32;
    constexpr int RPW = 32 / G;
    uint32_t tasks = 0;
    for (int i = 0; i < g.count; i++) {
        tasks += (g.item[i].n + RPW - 1) / RPW * (MOE ? g.item[i].rows * g.item[i].id_r : 1);
        g.task_end[i] = tasks;
    }
    const size_t smem = BAR_BYTES + (size_t)FAST_WARPS * 2 * Blk<FMT>::STAGE + g.act_bytes + (EARLY ? pend_bytes(M) : 0);
    static DynamicSmemOptIn opted;
    if (cudaError_t e = opted.raise((const void *)kern, smem); e != cudaSuccess) return e;
    // resident CTAs per SM for this shared-memory size (a handful of sizes occur: remembered per device)
    static OccupancyCache occupancy;
    int ctas_per_sm = 1;
    if (cudaError_t e = occupancy.get(kern, FAST_THREADS, smem, &ctas_per_sm); e != cudaSuccess) return e;
    // Leave one CTA slot per SM to the next kernel of the stream: under programmatic dependent
    // launch its CTAs move in while this kernel still runs and fill their rings, so the weight
    // stream does not stop at the kernel boundary.
    int per_sm = ctas_per_sm >= 4 ? ctas_per_sm - 1 : ctas_per_sm;
    // Early mode with parked results (one or two rows): a kernel computes all of its tasks without waiting
    // for the kernel in front, so consecutive launches run side by side as long as each leaves room for
    // the next ones. One small CTA per SM and kernel (two for two rows) measured best: up to five
    // kernels share an SM and the weight stream never stops at a kernel boundary.
    if (EARLY) per_sm = M == 1 ? 1 : (ctas_per_sm < 2 ? ctas_per_sm : 2);
    if (g_cta_cap > 0) per_sm = g_cta_cap < ctas_per_sm ? g_cta_cap : ctas_per_sm;
    // every SM gets the same number of CTAs and every CTA the same share of the tasks
    uint32_t grid = (uint32_t)sm_count * (uint32_t)per_sm;
    const uint32_t useful = (tasks + FAST_WARPS - 1) / FAST_WARPS;
    if (grid > useful) grid = useful;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(FAST_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, g);
}

template <int FMT, int M, int G>
static cudaError_t launch_fast(GemvGroup &g, int sm_count, bool pdl, cudaStream_t stream) {
    if (g.count > 1) return launch_fast_n<FMT, M, G, GEMV_GROUP_MAX>(g, sm_count, pdl, stream);
    GemvSingle one;
    one.item[0] = g.item[0];
    one.act_off[0] = g.act_off[0];
    one.act_copy[0] = g.act_copy[0];
    one.count = 1;
    one.act_bytes = g.act_bytes;
    return launch_fast_n<FMT, M, G, 1>(one, sm_count, pdl, stream);
}

template <int FMT, int M> static cudaError_t launch_fast_g(GemvGroup &a, int sm, bool pdl, cudaStream_t s) {
    const uint32_t nblk = a.item[0].k / QK;
    if (nblk <= 8) return launch_fast<FMT, M, 8>(a, sm, pdl, s);
    if (nblk <= 16) return launch_fast<FMT, M, 16>(a, sm, pdl, s);
    return launch_fast<FMT, M, 32>(a, sm, pdl, s);
}

static size_t stage_bytes(int fmt) {
    return fmt == FMT_Q4K ? Blk<FMT_Q4K>::STAGE : fmt == FMT_Q5K ? Blk<FMT_Q5K>::STAGE : Blk<FMT_Q6K>::STAGE;
}

// Any K that is a multiple of 256, as long as the rings and the activation records fit in shared memory.
bool qgemv_kq_fast_shape_ok(int fmt, uint32_t rows, uint32_t k) {
    if (fmt != FMT_Q4K && fmt != FMT_Q5K && fmt != FMT_Q6K) return false;
    if (rows < 1 || rows > 8 || k % QK != 0 || k < QK) return false;
    const size_t warps = rows <= 2 ? 4 : 8;
    const size_t stage = stage_bytes(fmt);
    return BAR_BYTES + warps * 2 * stage + (size_t)rows * (k / QK) * REC + pend_bytes((int)rows) <= 227 * 1024 - 256;
}

bool qgemv_kq_fast_supported(int fmt, const GemvArgs &a) {
    return qgemv_kq_fast_shape_ok(fmt, a.rows, a.k) && ((uintptr_t)a.w & 15) == 0;
}

bool qgemv_q4k_fast_supported(const GemvArgs &a) { return qgemv_kq_fast_supported(FMT_Q4K, a); }

template <int FMT> static cudaError_t launch_fmt(GemvGroup &a, int sm_count, bool pdl, cudaStream_t s) {
    switch (a.item[0].rows) {
        case 1: return launch_fast_g<FMT, 1>(a, sm_count, pdl, s);
        case 2: return launch_fast_g<FMT, 2>(a, sm_count, pdl, s);
        case 3: return launch_fast_g<FMT, 3>(a, sm_count, pdl, s);
        case 4: return launch_fast_g<FMT, 4>(a, sm_count, pdl, s);
        case 5: return launch_fast_g<FMT, 5>(a, sm_count, pdl, s);
        case 6: return launch_fast_g<FMT, 6>(a, sm_count, pdl, s);
        case 7: return launch_fast_g<FMT, 7>(a, sm_count, pdl, s);
        case 8: return launch_fast_g<FMT, 8>(a, sm_count, pdl, s);
        default: return cudaErrorInvalidValue;
    }
}

// Shared memory the activation records of a group need; distinct sources only.
static void plan_group_acts(GemvGroup &g) {
    const uint32_t bytes = g.item[0].rows * (g.item[0].k / QK) * REC;
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

size_t qgemv_kq_group_smem(int fmt, GemvGroup &g) {
    plan_group_acts(g);
    const size_t warps = g.item[0].rows <= 2 ? 4 : 8;
    const size_t stage = stage_bytes(fmt);
    return BAR_BYTES + warps * 2 * stage + g.act_bytes + pend_bytes((int)g.item[0].rows);
}

cudaError_t launch_qgemv_kq_group(int fmt, GemvGroup &g, int sm_count, bool pdl, cudaStream_t s) {
    if (g.count < 1 || g.count > GEMV_GROUP_MAX) return cudaErrorInvalidValue;
    plan_group_acts(g);
    return fmt == FMT_Q6K ? launch_fmt<FMT_Q6K>(g, sm_count, pdl, s)
                          : fmt == FMT_Q5K ? launch_fmt<FMT_Q5K>(g, sm_count, pdl, s) : launch_fmt<FMT_Q4K>(g, sm_count, pdl, s);
}

bool qgemv_kq_moe_shape_ok(int fmt, uint32_t tokens, uint32_t k) {
    if (fmt != FMT_Q4K && fmt != FMT_Q5K && fmt != FMT_Q6K) return false;
    if (tokens < 1 || tokens > 8 || k % QK != 0 || k < QK) return false;
    const size_t stage = stage_bytes(fmt);
    return BAR_BYTES + (size_t)Shape<1>::WARPS * 2 * stage + (size_t)tokens * (k / QK) * REC + pend_bytes(1) <= 227 * 1024 - 256;
}

template <int FMT, int G> static cudaError_t launch_moe_g(const GemvArgs &a, int sm_count, bool pdl, cudaStream_t s) {
    GemvSingle one{};
    one.item[0] = a;
    one.act_copy[0] = 1;
    one.count = 1;
    one.act_bytes = a.rows * (a.k / QK) * REC;
    return launch_fast_n<FMT, 1, G, 1, true>(one, sm_count, pdl, s);
}

template <int FMT> static cudaError_t launch_moe(const GemvArgs &a, int sm_count, bool pdl, cudaStream_t s) {
    const uint32_t nblk = a.k / QK;
    if (nblk <= 8) return launch_moe_g<FMT, 8>(a, sm_count, pdl, s);
    if (nblk <= 16) return launch_moe_g<FMT, 16>(a, sm_count, pdl, s);
    return launch_moe_g<FMT, 32>(a, sm_count, pdl, s);
}

cudaError_t launch_qgemv_kq_moe(int fmt, const GemvArgs &a, int sm_count, bool pdl, cudaStream_t s) {
    if (!qgemv_kq_moe_shape_ok(fmt, a.rows, a.k) || !a.ids || a.id_r == 0 || a.id_e == 0 || ((uintptr_t)a.w & 15) || (a.id_stride & 15))
        return cudaErrorInvalidValue;
    if ((uint64_t)a.rows * a.id_r * ((a.n + 3) / 4) >= (1ull << 31)) return cudaErrorInvalidValue;  // 32-bit task index
    return fmt == FMT_Q6K ? launch_moe<FMT_Q6K>(a, sm_count, pdl, s)
                          : fmt == FMT_Q5K ? launch_moe<FMT_Q5K>(a, sm_count, pdl, s) : launch_moe<FMT_Q4K>(a, sm_count, pdl, s);
}

cudaError_t launch_qgemv_kq_fast(int fmt, const GemvArgs &a, int sm_count, bool pdl, cudaStream_t s) {
    GemvGroup g{};
    g.count = 1;
    g.item[0] = a;
    return launch_qgemv_kq_group(fmt, g, sm_count, pdl, s);
}

cudaError_t launch_qgemv_q4k_fast(const GemvArgs &a, int sm_count, bool pdl, cudaStream_t s) {
    return launch_qgemv_kq_fast(FMT_Q4K, a, sm_count, pdl, s);
}

}  // namespace lb

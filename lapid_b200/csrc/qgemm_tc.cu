// Prefill GEMM on the 5th-generation tensor cores: out[m, n] = sum_k A[m, k] * dequant(W)[n, k] for
// Q4_K and Q6_K weights, bf16 operands, f32 accumulation in tensor memory.
//
// Reference semantics: lapid-cpu's path for more than 8 rows multiplies f32 activations by the
// dequantized f32 weights (crates/lapid-cpu/src/matmul/qdeq.rs:57-123); lapid-cuda's tensor-core
// kernel rounds both operands to f16 (crates/lapid-cuda/src/codegen/kquant.rs:335-519). Here both
// operands are rounded to bf16 (weights: bf16 of lapid-quant's f32 value -- Q4_K d1*q - m1 computed
// with one fused multiply-add, Q6_K d*sc*(q-32), exact in f32), products are exact and sums are
// f32, so the result differs from the f32 reference by the operand rounding only (2^-9 relative
// per operand).
//
// One CTA computes a 128*NT (weight rows) x MT (activation rows, 64/128/256/512) output tile, K in
// steps of 64 (one Q4_K "pair": 32 bytes of quants = two 32-element sub-blocks):
//   warp 0     one lane drives TMA for the activations: per k-step a 128-byte swizzled 2-D copy
//              of the bf16 activation tile (`cp.async.bulk.tensor.2d`, each CTA loads its own copy)
//   warp 18    one lane drives TMA for the weights: per super-block a 2-D tensor-map copy of the
//              tile rows' packed blocks (144 bytes; Q6_K: 224 bytes around the 2-byte aligned 210),
//              one super-block ahead of its consumers; Q6_K rows that are not 16-byte multiples
//              are copied row by row with the plain bulk copy by all lanes of the warp
//   warp 1     allocates tensor memory; one lane issues `tcgen05.mma` (M=128, N=MT, K=16, four
//              per k-step and accumulator) on shared-memory descriptors and commits to mbarriers
//   warps 2-17 dequantize to bf16 into the 128-byte-swizzled K-major layout the tensor core reads.
//              Q4_K: thread (row, half) expands one 32-element sub-block per k-step (NT = 1: warps
//              2-9 the even k-steps, 10-17 the odd ones; NT = 2: the two groups own the two 128-row
//              sub-tiles). Q6_K: 16 lanes share a row, lane = four weights. Afterwards warps 2-9
//              (NT = 2: all) are the epilogue: `tcgen05.ld` 32 lanes x 32 columns at a time,
//              optional `+ extra`, coalesced f32 stores
// The weight tile is the M side of the MMA and the activations the N side, so 64 prefill rows
// use a 128x64 instruction at full rate instead of padding to 128 rows.
// Tile shapes: NT = 2 at MT = 256 (two accumulators, all 512 columns of tensor memory) halves the
// activation traffic per flop; MT = 512 with NT = 1 halves the dequantization per flop instead
// (chosen for Q6_K by waves of tiles over the SMs). Launches with too few tiles for the SMs split K
// over gridDim.z: partial tiles go to a scratch area and a second kernel sums them in order.
// PAIR (off by default): two CTAs of a cluster as one `cta_group::2` unit, each loading half of the
// activation tile; measured slower than the single-CTA 256x256 tile.
// Every mbarrier wait is bounded: a wait that gives up sets a bit in the host-visible status
// word, the roles fall through to the end, tensor memory is released and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstring>

#include "common.cuh"
#include "kernels.h"

namespace lb {

namespace tc {

constexpr int TN = 128;            // weight rows per tile
constexpr int KS = 64;             // k per stage
constexpr int Q6K_BOX = 224;       // Q6_K: bytes staged per row and super-block (210 from a 2-byte aligned start, see below)
constexpr int B_BYTES = TN * 128;  // bf16 weight tile of one stage
constexpr int THREADS = 608;       // 19 warps
constexpr int DEQ_WARPS = 16;      // two groups of eight: even and odd k-steps
constexpr int GROUP_WARPS = 8;
constexpr uint32_t SPIN_LIMIT = 1u << 24;

// MT activation rows x (NT * 128) weight rows per CTA. NT = 2 keeps two accumulators (all 512
// columns of tensor memory at MT = 256) so that one activation tile feeds twice the weights: the
// bf16 activation tile is the larger part of what an SM pulls from L2 per k-step.
// PAIR: two CTAs of a cluster run as one `cta_group::2` tensor-core unit: each dequantizes its own
// 128*NT weight rows and loads only HALF of the activation tile (the instruction reads both CTAs'
// halves), which halves the activation traffic from L2 and leaves room for a third stage.
template <int FMT, int MT, int NT, bool PAIR = false> struct Cfg {
    static constexpr int STAGES = PAIR ? 3 : ((NT == 2 || MT == 512) ? 2 : (MT == 256 ? 3 : 4));
    static constexpr int A_BYTES = (PAIR ? MT / 2 : MT) * 128;
    static constexpr int W_BYTES = NT * B_BYTES;
    static constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
    static constexpr int ROW_BYTES = FMT == FMT_Q4K ? Q4K_BYTES : FMT == FMT_Q5K ? Q5K_BYTES : Q6K_BOX;  // packed bytes staged per row and super-block
    static constexpr int RAW_BYTES = TN * ROW_BYTES;                         // one 128-row sub-tile: 18432 / 28672
    static constexpr int RAW = NT * RAW_BYTES;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 2 * RAW + 256 /*barriers*/ + 1024 /*alignment slack*/;
};

__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(bar)) : "memory");
}
// Bounded wait. A waiter that is not on the critical path sleeps between polls so that it does not
// take issue slots from the dequantizing warps.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t sleep_ns = 0) {
    for (uint32_t spin = 0; spin < SPIN_LIMIT; spin++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(s32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
        if (sleep_ns) __nanosleep(sleep_ns);
    }
    return false;
}

// Two f32 lanes in one 64-bit register pair: Blackwell's packed f32 pipe halves the instruction
// count of the dequantization.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
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
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// {lo, hi} f32 -> packed bf16x2 with lo in the low half
__device__ __forceinline__ uint32_t to_bf16x2(uint64_t v) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     s32(dst)),
                 "l"((uint64_t)map), "r"(x), "r"(y), "r"(s32(bar))
                 : "memory");
}

// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}
// ---- the same for a pair of CTAs (`cta_group::2`); `cluster_addr` may name a barrier of either CTA
__device__ __forceinline__ void mma_bf16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_commit_pair(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}
// the shared::cluster address of `p` in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t cluster_addr_of(const void *p, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(s32(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// bounded wait with cluster-scope acquire: the arrival comes from the other CTA of the pair
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t *bar, uint32_t parity, uint32_t sleep_ns = 0) {
    for (uint32_t spin = 0; spin < SPIN_LIMIT; spin++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(s32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
        if (sleep_ns) __nanosleep(sleep_ns);
    }
    return false;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// f32 bits of (2^23 + byte `sel` of w): the byte planted in the mantissa by one PRMT
__device__ __forceinline__ float biased(uint32_t w, uint32_t sel) { return __uint_as_float(__byte_perm(w, 0x4B000000u, sel)); }

template <int FMT, int MT, int NT, bool PAIR>
__global__ void __launch_bounds__(THREADS, 1)
qgemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, GemmTcArgs p) {
    using C = Cfg<FMT, MT, NT, PAIR>;
    constexpr int RAW_BYTES = C::RAW_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *stage0 = smem;
    uint8_t *raw0 = smem + C::STAGES * C::STAGE_BYTES;
    uint64_t *bars = (uint64_t *)(raw0 + 2 * C::RAW);
    uint64_t *full_a = bars, *full_b = bars + C::STAGES, *empty = bars + 2 * C::STAGES;
    uint64_t *raw_full = bars + 3 * C::STAGES, *raw_empty = raw_full + 2, *acc_full = raw_full + 4;
    uint32_t *tmem_slot = (uint32_t *)(acc_full + 1);
    uint64_t *peer_ready = acc_full + 2;  // PAIR, leader CTA: the other CTA's operands of a stage are in place
    uint32_t cta_rank = 0;
    if constexpr (PAIR) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cta_rank));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n0 = blockIdx.x * (TN * NT), m0 = blockIdx.y * MT;
    // Expert-indexed launch (Kernel::MatMulId, moe.cu): the activation tiles are runs of (token, slot)
    // pairs grouped by expert; the weights are the dense stack [experts * n, k], so a tile's weight
    // rows start at expert * n. Tiles past the last used one have no expert.
    uint32_t wrow0 = 0;
    if (p.tile_expert) {
        const int32_t e = p.tile_expert[blockIdx.y];
        if (e < 0) return;  // before any barrier or tensor-memory allocation
        wrow0 = (uint32_t)e * p.n;
    }
    // split-K: CTA z of gridDim.z takes the super-blocks [kb0, kb0 + nblk) of K and writes a partial tile
    const uint32_t nblk_total = p.k / QK, per_split = (nblk_total + gridDim.z - 1) / gridDim.z;
    const uint32_t kb0 = blockIdx.z * per_split;
    const uint32_t nblk = min(per_split, nblk_total - kb0), ksteps = nblk * (QK / KS);

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(full_a + s, 1);
            mbar_init(full_b + s, NT == 2 ? DEQ_WARPS : GROUP_WARPS);
            mbar_init(empty + s, 1);
        }
        for (int r = 0; r < 2; r++) {
            mbar_init(raw_full + r, 1);
            mbar_init(raw_empty + r, DEQ_WARPS);
        }
        mbar_init(acc_full, 1);
        if constexpr (PAIR)
            for (int s = 0; s < C::STAGES; s++) mbar_init(peer_ready + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (PAIR) {  // the same warp of both CTAs: a pair-wide allocation of the same columns
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"((uint32_t)(MT * NT)) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"((uint32_t)(MT * NT)) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();  // both CTAs' barriers exist before either one signals the other
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    bool healthy = true;

    if (warp == 0) {
        // ---------------- TMA producer, activation tiles: one 128-byte-swizzled box per k-step
        if (lane == 0) {
            for (uint32_t ks = 0; ks < ksteps && healthy; ks++) {
                const uint32_t s = ks % C::STAGES, u = ks / C::STAGES;
                if (!mbar_wait(empty + s, (u & 1) ^ 1, 64)) { healthy = false; break; }
                mbar_expect_tx(full_a + s, C::A_BYTES);
                if constexpr (PAIR) {  // this CTA's half of the activation tile
                    tma_load_2d(stage0 + s * C::STAGE_BYTES + C::W_BYTES, &map_a, (int)(kb0 * QK + ks * KS), (int)(m0 + (MT / 2) * cta_rank), full_a + s);
                } else {
#pragma unroll
                    for (int h = 0; h < (MT + 255) / 256; h++)  // a box holds at most 256 rows
                        tma_load_2d(stage0 + s * C::STAGE_BYTES + C::W_BYTES + h * 256 * 128, &map_a, (int)(kb0 * QK + ks * KS), (int)(m0 + 256 * h),
                                    full_a + s);
                }
            }
            if (!healthy && p.status) atomicOr(p.status, 2);
        }
    } else if (warp == 18 && FMT == FMT_Q6K && ((nblk_total * Q6K_BYTES) & 15u) != 0) {
        // ---------------- packed Q6_K weights whose rows are not a multiple of 16 bytes (K not a
        // multiple of 2048, e.g. the K/8 shard of a row-parallel projection): no tensor map can
        // describe them, so every lane copies rows of the tile with the plain bulk copy, each from
        // the 16-byte boundary below its block (the consumers compute the same per-row offset)
        const uint32_t rows_valid = min((uint32_t)TN, p.n > n0 ? p.n - n0 : 0u);
        const uint64_t pitch = (uint64_t)nblk_total * Q6K_BYTES;
        const uint64_t end16 = ((uint64_t)(uintptr_t)p.w + (uint64_t)p.n * pitch + 15) & ~(uint64_t)15;  // never read past the matrix's last 16-byte line
        auto copy_of = [&](uint32_t rr, uint32_t b, uint64_t &src) -> uint32_t {
            src = ((uint64_t)(uintptr_t)p.w + (uint64_t)(n0 + rr) * pitch + (uint64_t)(kb0 + b) * Q6K_BYTES) & ~(uint64_t)15;
            return (uint32_t)min((uint64_t)Q6K_BOX, end16 - src);
        };
        for (uint32_t b = 0; b < nblk && healthy; b++) {
            const uint32_t r = b & 1, ur = b >> 1;
            if (!mbar_wait(raw_empty + r, (ur & 1) ^ 1, 64)) { healthy = false; break; }
            if (lane == 0 && rows_valid) {
                uint64_t src;
                mbar_expect_tx(raw_full + r, (rows_valid - 1) * Q6K_BOX + copy_of(rows_valid - 1, b, src));  // only the last row can be short
            }
            __syncwarp();
            for (uint32_t rr = lane; rr < rows_valid; rr += 32) {
                uint64_t src;
                const uint32_t bytes = copy_of(rr, b, src);
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 s32(raw0 + r * C::RAW + rr * Q6K_BOX)),
                             "l"(src), "r"(bytes), "r"(s32(raw_full + r))
                             : "memory");
            }
        }
        if (!healthy && lane == 0 && p.status) atomicOr(p.status, 32);
    } else if (warp == 18) {
        // ---------------- TMA producer, packed weights: one super-block of every row of the tile
        // per copy, a whole super-block (four k-steps) ahead of the dequantizing warps
        if (lane == 0) {
            for (uint32_t b = 0; b < nblk && healthy; b++) {
                const uint32_t r = b & 1, ur = b >> 1;
                if (!mbar_wait(raw_empty + r, (ur & 1) ^ 1, 64)) { healthy = false; break; }
                mbar_expect_tx(raw_full + r, C::RAW);
#pragma unroll
                for (int t = 0; t < NT; t++)
                    tma_load_2d(raw0 + r * C::RAW + t * RAW_BYTES, &map_w,
                                FMT == FMT_Q6K ? (int)(((kb0 + b) * Q6K_BYTES) & ~15u) : (int)((kb0 + b) * C::ROW_BYTES), (int)(wrow0 + n0 + t * TN),
                                raw_full + r);
            }
            if (!healthy && p.status) atomicOr(p.status, 32);
        }
    } else if (warp == 1 && PAIR) {
        // ---------------- MMA issuer of a CTA pair. The leader (rank 0) issues for both CTAs: M = 256
        // (128 weight rows from each CTA's tile), N = MT (each CTA holds MT / 2 activation rows), the
        // accumulators land in each CTA's own tensor memory. The other CTA's issuer warp only reports
        // when its operands of a stage are in place. Completion is committed to both CTAs' barriers.
        if (lane == 0) {
            const uint32_t peer = cta_rank ^ 1;
            if (cta_rank == 0) {
                constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MT >> 3) << 17) | ((uint32_t)((2 * TN) >> 4) << 24);
                for (uint32_t ks = 0; ks < ksteps && healthy; ks++) {
                    const uint32_t s = ks % C::STAGES, u = ks / C::STAGES;
                    if (!mbar_wait(full_a + s, u & 1, 32) || !mbar_wait(full_b + s, u & 1, 32) || !mbar_wait_cluster(peer_ready + s, u & 1, 32)) {
                        healthy = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t wt = s32(stage0 + s * C::STAGE_BYTES), at = wt + C::W_BYTES;
#pragma unroll
                    for (int t = 0; t < NT; t++)
#pragma unroll
                        for (int kk = 0; kk < KS / 16; kk++)
                            mma_bf16_pair(tmem_base + t * MT, smem_desc(wt + t * B_BYTES + kk * 32), smem_desc(at + kk * 32), idesc, (ks | kk) ? 1u : 0u);
                    mma_commit_pair(s32(empty + s));
                    mma_commit_pair(cluster_addr_of(empty + s, peer));
                }
                mma_commit_pair(s32(acc_full));
                mma_commit_pair(cluster_addr_of(acc_full, peer));
                if (!healthy && p.status) atomicOr(p.status, 4);
            } else {
                for (uint32_t ks = 0; ks < ksteps && healthy; ks++) {
                    const uint32_t s = ks % C::STAGES, u = ks / C::STAGES;
                    if (!mbar_wait(full_a + s, u & 1, 32) || !mbar_wait(full_b + s, u & 1, 32)) { healthy = false; break; }
                    mbar_arrive_cluster(cluster_addr_of(peer_ready + s, peer));
                }
                if (!healthy && p.status) atomicOr(p.status, 4);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            // D f32, A and B bf16, both K-major, M = 128, N = MT
            constexpr int MMA_N = MT > 256 ? 256 : MT;  // an instruction takes at most 256 columns: MT = 512 issues two
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MMA_N >> 3) << 17) | ((uint32_t)(TN >> 4) << 24);
            for (uint32_t ks = 0; ks < ksteps && healthy; ks++) {
                const uint32_t s = ks % C::STAGES, u = ks / C::STAGES;
                if (!mbar_wait(full_a + s, u & 1, 32) || !mbar_wait(full_b + s, u & 1, 32)) { healthy = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t wt = s32(stage0 + s * C::STAGE_BYTES), at = wt + C::W_BYTES;
#pragma unroll
                for (int t = 0; t < NT; t++)
#pragma unroll
                    for (int kk = 0; kk < KS / 16; kk++)
#pragma unroll
                        for (int h = 0; h < MT / MMA_N; h++)
                            mma_bf16(tmem_base + t * MT + h * MMA_N, smem_desc(wt + t * B_BYTES + kk * 32),
                                     smem_desc(at + h * MMA_N * 128 + kk * 32), idesc, (ks | kk) ? 1u : 0u);
                mma_commit(empty + s);  // the stage may be refilled once these MMAs have read it
            }
            mma_commit(acc_full);
            if (!healthy && p.status) atomicOr(p.status, 4);
        }
    } else {
        // ---------------- dequantize: thread = (weight row of the tile, which 32 of the 64 k); the
        // first eight warps take the even k-steps, the other eight the odd ones, so that a warp
        // has two MMA periods for one k-step and the groups' waits overlap
        // (NT = 2: the two groups own the two 128-row sub-tiles instead and every warp does every k-step)
        const int dw = (warp - 2) & 7, grp = (warp - 2) >> 3;
        const int row = 32 * (dw & 3) + lane, half = dw >> 2;
        const int sub = NT == 2 ? grp : 0;        // weight sub-tile of this thread
        float d1[4], m1[4];                       // sub-block scales of this thread's pairs of the current super-block
        for (uint32_t ks = (NT == 2 ? 0 : grp); ks < ksteps && healthy; ks += (NT == 2 ? 1 : 2)) {
            const uint32_t s = ks % C::STAGES, u = ks / C::STAGES;
            const uint32_t b = ks >> 2, pp = ks & 3, r = b & 1, ur = b >> 1;
            if constexpr (FMT == FMT_Q6K) {
                // Q6_K (NT = 1): a super-block is ql[128] | qh[64] | int8 sc[16] | f16 d = 210 bytes, so it
                // starts on a 2-byte boundary only; the copy starts at the 16-byte boundary below it and
                // takes 224 bytes per row. 16 lanes share one weight row of the k-step: lane j expands the
                // four weights 4j..4j+3 of its 64 (16-bit shared loads, conflict-free along the row), a
                // warp does two rows per pass and 16 rows per k-step.
                //   k-step pp of the block: half nh = pp >> 1 of the 256, nibble hi = pp & 1; the first 32
                //   weights come from ql[64 nh + l], the second 32 from ql[64 nh + 32 + l]; the two high
                //   bits from qh[32 nh + l] >> 2 * (2 hi + h); scale sc[8 nh + 2 (2 hi + h) + l / 16]
                //   (crates/lapid-quant/src/kquant.rs:375-396). d * sc * (q - 32) is exact in f32.
                if (pp < 2 && !mbar_wait(raw_full + r, ur & 1)) { healthy = false; break; }
                if (!mbar_wait(empty + s, (u & 1) ^ 1)) { healthy = false; break; }
                const uint32_t j = lane & 15, h = j >> 3, jj = j & 7, nh = pp >> 1, hi = pp & 1;
                const uint64_t pitch = (uint64_t)nblk_total * Q6K_BYTES, wbase = (uint64_t)(uintptr_t)p.w + (uint64_t)(kb0 + b) * Q6K_BYTES;
                const uint64_t unbias32 = pack2(-8388640.0f, -8388640.0f);  // -(2^23 + 32)
#pragma unroll 2
                for (int pass = 0; pass < 8; pass++) {
                    const int rw = 16 * dw + 2 * pass + (lane >> 4);
                    // where the block starts inside its 224 staged bytes: the distance of its address from
                    // the 16-byte boundary below it (the same for every row when the row pitch is a multiple of 16)
                    const uint32_t skew = (uint32_t)((wbase + (uint64_t)(n0 + rw) * pitch) & 15u);
                    const uint8_t *blk = raw0 + r * C::RAW + rw * Q6K_BOX + skew;
                    const uint16_t *ql = (const uint16_t *)(blk + 64 * nh + 32 * h + 4 * jj);
                    const uint16_t *qh = (const uint16_t *)(blk + 128 + 32 * nh + 4 * jj);
                    const uint32_t wl = (uint32_t)ql[0] | ((uint32_t)ql[1] << 16), wh = (uint32_t)qh[0] | ((uint32_t)qh[1] << 16);
                    const uint32_t q = ((wl >> (4 * hi)) & 0x0F0F0F0Fu) | (((wh >> (2 * (2 * hi + h))) & 0x03030303u) << 4);
                    const float sc = (float)(int)*(const int8_t *)(blk + 192 + 8 * nh + 2 * (2 * hi + h) + (jj >> 2));
                    const float sd = half_bits_to_float(*(const uint16_t *)(blk + 208)) * sc;
                    const uint64_t sd2 = pack2(sd, sd);
                    const uint64_t q01 = add2(pack2(biased(q, 0x7440u), biased(q, 0x7441u)), unbias32);
                    const uint64_t q23 = add2(pack2(biased(q, 0x7442u), biased(q, 0x7443u)), unbias32);
                    const uint32_t o0 = to_bf16x2(mul2(sd2, q01)), o1 = to_bf16x2(mul2(sd2, q23));
                    uint8_t *dst = stage0 + s * C::STAGE_BYTES + rw * 128;
                    const int chunk = (int)(j >> 1) ^ (rw & 7);
                    *(uint2 *)(dst + 16 * chunk + 8 * (j & 1)) = make_uint2(o0, o1);
                }
                if (pp >= 2) {  // this warp's last read of the block's packed bytes
                    __syncwarp();
                    if (lane == 0) mbar_arrive(raw_empty + r);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> tensor-core reads
                __syncwarp();
                if (lane == 0) mbar_arrive(full_b + s);
                continue;
            }
            const uint8_t *blk = raw0 + r * C::RAW + sub * RAW_BYTES + row * C::ROW_BYTES;
            if (NT == 2 ? pp == 0 : pp < 2) {  // first k-step of this thread in the block
                if (!mbar_wait(raw_full + r, ur & 1)) { healthy = false; break; }
                const uint4 h = *(const uint4 *)blk;
                const float d = half_bits_to_float(h.x & 0xffff), dmin = half_bits_to_float(h.x >> 16);
                const float nd = d * -8388608.0f, ndmin = dmin * -8388608.0f;
                const uint32_t w0 = h.y, w1 = h.z, w2 = h.w;
                const uint32_t sc_lo = w0 & 0x3F3F3F3Fu, mn_lo = w1 & 0x3F3F3F3Fu;
                const uint32_t sc_hi = (w2 & 0x0F0F0F0Fu) | (((w0 >> 6) & 0x03030303u) << 4);
                const uint32_t mn_hi = ((w2 >> 4) & 0x0F0F0F0Fu) | (((w1 >> 6) & 0x03030303u) << 4);
                // pair q: sub-block 2q + half = byte 2*(q&1) + half of the lo (q < 2) / hi words
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint32_t sel = 0x7440u + 2 * (q & 1) + half;
                    d1[q] = fmaf(d, biased(q < 2 ? sc_lo : sc_hi, sel), nd);        // d * sc, exact (see qgemv_q4k.cu)
                    m1[q] = fmaf(dmin, biased(q < 2 ? mn_lo : mn_hi, sel), ndmin);  // dmin * m, exact
                }
            }
            // Q5_K: Q4_K's block with the fifth bits qh[32] between the header and the nibbles; bit s of qh[l]
            // belongs to element 32 s + l (crates/lapid-quant/src/kquant.rs:355-373)
            constexpr int QS = FMT == FMT_Q5K ? 48 : 16;
            const uint4 qa = *(const uint4 *)(blk + QS + 32 * pp), qb = *(const uint4 *)(blk + QS + 16 + 32 * pp);
            uint4 ha = make_uint4(0, 0, 0, 0), hb = ha;
            if constexpr (FMT == FMT_Q5K) {
                ha = *(const uint4 *)(blk + 16);
                hb = *(const uint4 *)(blk + 32);
            }
            if (NT == 2 ? pp == 3 : pp >= 2) {  // this thread's last read of the block's packed bytes
                __syncwarp();
                if (lane == 0) mbar_arrive(raw_empty + r);
            }
            const float sd = pp == 0 ? d1[0] : pp == 1 ? d1[1] : pp == 2 ? d1[2] : d1[3];
            const float nm = -(pp == 0 ? m1[0] : pp == 1 ? m1[1] : pp == 2 ? m1[2] : m1[3]);
            const uint64_t sd2 = pack2(sd, sd), nm2 = pack2(nm, nm), unbias = pack2(-8388608.0f, -8388608.0f);
            uint32_t v[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
            if (half) {
#pragma unroll
                for (int i = 0; i < 8; i++) v[i] >>= 4;
            }
            if constexpr (FMT == FMT_Q5K) {
                const uint32_t hq[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
#pragma unroll
                for (int i = 0; i < 8; i++) v[i] = (v[i] & 0x0F0F0F0Fu) | (((hq[i] >> (2 * pp + half)) & 0x01010101u) << 4);
            }
            if (!mbar_wait(empty + s, (u & 1) ^ 1)) { healthy = false; break; }
            uint8_t *dst = stage0 + s * C::STAGE_BYTES + sub * B_BYTES + row * 128;
#pragma unroll
            for (int c = 0; c < 4; c++) {  // 16-byte chunk = 8 consecutive k = two packed words
                uint32_t o[4];
#pragma unroll
                for (int w = 0; w < 2; w++) {
                    const uint32_t t = v[2 * c + w] & (FMT == FMT_Q5K ? 0x1F1F1F1Fu : 0x0F0F0F0Fu);
                    // y = sd * q - m1 with one rounding, two elements per instruction
                    const uint64_t q01 = add2(pack2(biased(t, 0x7440u), biased(t, 0x7441u)), unbias);
                    const uint64_t q23 = add2(pack2(biased(t, 0x7442u), biased(t, 0x7443u)), unbias);
                    o[2 * w] = to_bf16x2(fma2(sd2, q01, nm2));
                    o[2 * w + 1] = to_bf16x2(fma2(sd2, q23, nm2));
                }
                const int chunk = (4 * half + c) ^ (row & 7);
                *(uint4 *)(dst + 16 * chunk) = make_uint4(o[0], o[1], o[2], o[3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> tensor-core reads
            __syncwarp();
            if (lane == 0) mbar_arrive(full_b + s);
        }
        if (!healthy && lane == 0 && p.status) atomicOr(p.status, 8);

        // ---------------- epilogue: TMEM lane = weight row, column = activation row
        if (NT == 1 && grp != 0) {
            // with one accumulator the second group has no epilogue share
        } else if (healthy && mbar_wait(acc_full, 0)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int quarter = warp & 3;  // the TMEM lanes this warp may read
            const uint32_t n = n0 + sub * TN + 32 * quarter + lane;
            constexpr int COLS = MT / 2;   // each half of the epilogue warps takes half of the columns
            const int cbase = half * COLS;
#pragma unroll 1
            for (int c0 = 0; c0 < COLS; c0 += 32) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(sub * MT + cbase + c0);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                      "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                      "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                      "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (p.row_pair) {  // expert-indexed: tile-space row -> (token, slot) pair = output row; padding rows have none
                    const uint32_t mfirst = m0 + cbase + c0;
                    if (n < p.n) {
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const int32_t pair = p.row_pair[mfirst + j];
                            if (pair >= 0) p.out[p.out_off + (uint64_t)pair * p.n + n] = __uint_as_float(r[j]);
                        }
                    }
                } else if (n < p.n && p.partial) {  // split-K: this CTA's partial sums, [split][row][n]; summed by a second kernel
                    const uint32_t mfirst = m0 + cbase + c0;
                    float *prow = p.partial + ((size_t)blockIdx.z * p.rows + mfirst) * p.n + n;
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (mfirst + j < p.rows) prow[(size_t)j * p.n] = __uint_as_float(r[j]);
                } else if (n < p.n) {
                    // (batch, row) of the chunk's first activation row by one division, then by stepping
                    const uint32_t mfirst = m0 + cbase + c0;
                    uint32_t bt = mfirst / p.m, i = mfirst % p.m;
                    float *orow = p.out + p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)i * p.out_rs + n;
                    const float *erow = p.extra ? p.extra + p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)i * p.ex_s1 + (int64_t)n * p.ex_s2 : nullptr;
                    if (!erow && i + 32 <= p.m && mfirst + 32 <= p.rows) {  // the common case: 32 whole rows of one batch entry, no epilogue term
#pragma unroll
                        for (int j = 0; j < 32; j++) orow[(uint64_t)j * p.out_rs] = __uint_as_float(r[j]);
                        continue;
                    }
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        if (mfirst + j < p.rows) {
                            float v = __uint_as_float(r[j]);
                            if (erow) v += *erow;
                            *orow = v;
                        }
                        if (++i == p.m) {  // next batch entry
                            i = 0;
                            bt++;
                            orow = p.out + p.out_off + (uint64_t)bt * p.out_bs + n;
                            if (erow) erow = p.extra + p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)n * p.ex_s2;
                        } else {
                            orow += p.out_rs;
                            if (erow) erow += p.ex_s1;
                        }
                    }
                }
            }
        } else if (lane == 0 && p.status) {
            atomicOr(p.status, 16);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();  // neither CTA releases the pair's tensor memory (or exits) while the other still uses it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if constexpr (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(MT * NT)) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(MT * NT)) : "memory");
    }
}

// split-K second pass: out[m, n] = sum over the splits (in order) of their partial tiles (+ extra)
__global__ void __launch_bounds__(256) splitk_sum_kernel(GemmTcArgs p, uint32_t splits) {
    const uint64_t total = (uint64_t)p.rows * p.n;
    for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t m = (uint32_t)(e / p.n), n = (uint32_t)(e % p.n);
        float v = p.partial[e];
        for (uint32_t z = 1; z < splits; z++) v += p.partial[(size_t)z * total + e];
        const uint32_t bt = m / p.m, i = m % p.m;
        if (p.extra) v += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)i * p.ex_s1 + (int64_t)n * p.ex_s2];
        p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)i * p.out_rs + n] = v;
    }
}

// f32 activation rows (any row stride) -> contiguous bf16 [rows, k]: blockIdx.y = row (one division per
// thread, not per element), a thread converts eight consecutive elements (k is a multiple of 256);
// VEC: the rows are 16-byte aligned, so the loads are 128-bit.
template <bool VEC> __global__ void __launch_bounds__(256) a_to_bf16_kernel(GemmTcArgs p, __nv_bfloat16 *dst) {
  for (uint32_t r = blockIdx.y; r < p.rows; r += gridDim.y) {
    const void *srow = act_row(p.a, p.a_type, p.a_off, p.a_bs, p.a_rs, r, p.m);
    const float *src = (const float *)srow;  // (VEC: f32 rows only)
    uint4 *out = (uint4 *)(dst + (size_t)r * p.k);
    for (uint32_t c8 = blockIdx.x * blockDim.x + threadIdx.x; c8 < p.k / 8; c8 += gridDim.x * blockDim.x) {
        float v[8];
        if constexpr (VEC) {
            const float4 lo = ((const float4 *)src)[2 * c8], hi = ((const float4 *)src)[2 * c8 + 1];
            v[0] = lo.x, v[1] = lo.y, v[2] = lo.z, v[3] = lo.w, v[4] = hi.x, v[5] = hi.y, v[6] = hi.z, v[7] = hi.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = load_act(srow, 8 * c8 + i, p.a_type);
        }
        __nv_bfloat162 o[4];
#pragma unroll
        for (int i = 0; i < 4; i++) o[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        out[c8] = *(const uint4 *)o;
    }
  }
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

template <int FMT, int MT, int NT, bool PAIR = false>
static cudaError_t launch_mt(const GemmTcArgs &a, const CUtensorMap &mw, const CUtensorMap &ma, cudaStream_t stream, uint32_t splits = 1) {
    auto kern = qgemm_tc_kernel<FMT, MT, NT, PAIR>;
    using C = Cfg<FMT, MT, NT, PAIR>;
    static DynamicSmemOptIn opted;
    if (cudaError_t e = opted.raise((const void *)kern, C::SMEM); e != cudaSuccess) return e;
    dim3 grid((a.n + TN * NT - 1) / (TN * NT), (a.rows + MT - 1) / MT, splits);
    if (!PAIR) {
        kern<<<grid, THREADS, C::SMEM, stream>>>(mw, ma, a);
        return cudaGetLastError();
    }
    grid.x = (grid.x + 1) & ~1u;  // whole pairs: a CTA past the last weight row works on zero fill and stores nothing
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = C::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, mw, ma, a);
}

}  // namespace tc

static int g_tc_wide = -1;  // tuning: -1 choose, 0 never, 1 always use two accumulators at MT = 256
static int g_tc_tall = -1;  // tuning: -1 choose, 0 never, 1 always use 512-row activation tiles above 256 rows
static int g_tc_pair = 0;   // tuning: 1 = CTA pairs (cta_group::2) for the two-accumulator Q4_K tile
void qgemm_tc_set_pair(int v) { g_tc_pair = v; }
void qgemm_tc_set_wide(int v) { g_tc_wide = v; }
void qgemm_tc_set_tall(int v) { g_tc_tall = v; }

bool qgemm_tc_supported(int fmt, const GemmTcArgs &a) {
    if (a.k % QK != 0 || a.k < QK || a.rows < 1 || ((uintptr_t)a.w & 15) != 0 || tc::encode_fn() == nullptr) return false;
    return fmt == FMT_Q4K || fmt == FMT_Q5K || fmt == FMT_Q6K;
}

static uint32_t tc_block_bytes(int fmt) { return fmt == FMT_Q4K ? Q4K_BYTES : fmt == FMT_Q5K ? Q5K_BYTES : Q6K_BYTES; }
static uint32_t tc_box_bytes(int fmt) { return fmt == FMT_Q6K ? (uint32_t)tc::Q6K_BOX : tc_block_bytes(fmt); }
// the one-accumulator tile of a format by activation rows per CTA
template <int FMT> static cudaError_t launch_one_acc(uint32_t mt, const GemmTcArgs &a, const CUtensorMap &mw, const CUtensorMap &ma,
                                                     cudaStream_t stream, uint32_t ways = 1) {
    using namespace tc;
    return mt == 64 ? launch_mt<FMT, 64, 1>(a, mw, ma, stream, ways)
                    : mt == 128 ? launch_mt<FMT, 128, 1>(a, mw, ma, stream, ways)
                                : mt == 256 ? launch_mt<FMT, 256, 1>(a, mw, ma, stream, ways) : cudaErrorInvalidValue;
}

// How many ways K is split: only when the tiles would leave more than half of the SMs idle, never
// below two super-blocks per split, never more partial-sum scratch than SPLITK_SCRATCH_MAX.
constexpr size_t SPLITK_SCRATCH_MAX = (size_t)256 << 20;
static int g_tc_splitk = -1;  // tuning: -1 choose, 0/1 never, n > 1 always n (where K allows)
void qgemm_tc_set_splitk(int v) { g_tc_splitk = v; }
static uint32_t splitk_ways(uint32_t rows, uint32_t n, uint32_t k, int sm_count) {
    const uint32_t mt = rows <= 64 ? 64 : (rows <= 128 ? 128 : 256);
    const uint64_t tiles = (uint64_t)((n + tc::TN - 1) / tc::TN) * ((rows + mt - 1) / mt);
    const uint32_t nblk = k / QK;
    uint32_t ways = 1;
    if (g_tc_splitk > 1) ways = (uint32_t)g_tc_splitk;
    else if (g_tc_splitk < 0 && sm_count > 0 && tiles * 2 <= (uint64_t)sm_count) ways = (uint32_t)((uint64_t)sm_count / tiles);
    if (ways > nblk / 2) ways = nblk / 2;
    if (ways > 16) ways = 16;
    while (ways > 1 && (size_t)ways * rows * n * 4 > SPLITK_SCRATCH_MAX) ways--;
    // every split must own at least one super-block
    while (ways > 1 && (uint64_t)(ways - 1) * ((nblk + ways - 1) / ways) >= nblk) ways--;
    return ways < 1 ? 1 : ways;
}

// bf16 copy of the activations, then (16-byte aligned) the partial sums of a split-K launch
size_t qgemm_tc_scratch_bytes(uint32_t rows, uint32_t n, uint32_t k, int sm_count) {
    const size_t a_bytes = ((size_t)rows * k * 2 + 255) & ~(size_t)255;
    const uint32_t ways = splitk_ways(rows, n, k, sm_count);
    return a_bytes + (ways > 1 ? (size_t)ways * rows * n * 4 : 0);
}

bool qgemm_tc_moe_supported(int fmt, uint64_t experts, uint64_t n, uint64_t k, const void *w) {
    if (fmt != FMT_Q4K && fmt != FMT_Q5K && fmt != FMT_Q6K) return false;
    if (k % QK != 0 || k < QK || ((uintptr_t)w & 15) != 0 || tc::encode_fn() == nullptr) return false;
    const uint64_t pitch = k / QK * tc_block_bytes(fmt);
    // one tensor map over all experts' rows: rows of 16-byte multiples, no padding between the matrices
    return pitch % 16 == 0 && (n * pitch) % 256 == 0 && experts * n < (1ull << 31);
}

cudaError_t launch_qgemm_tc_moe(int fmt, const GemmTcArgs &a, uint32_t experts, uint32_t mt, void *a_bf16, cudaStream_t stream) {
    using namespace tc;
    if (a.rows == 0 || a.n == 0) return cudaSuccess;
    EncodeTiledFn enc = encode_fn();
    if (!enc || !a.tile_expert || !a.row_pair || a.rows % mt != 0) return cudaErrorInvalidValue;
    CUtensorMap mw, ma;
    {
        const uint32_t blk_bytes = tc_block_bytes(fmt);
        cuuint64_t dims[2] = {(cuuint64_t)(a.k / QK) * blk_bytes, (cuuint64_t)experts * a.n};
        cuuint64_t strides[1] = {(cuuint64_t)(a.k / QK) * blk_bytes};
        cuuint32_t box[2] = {(cuuint32_t)tc_box_bytes(fmt), TN};
        cuuint32_t es[2] = {1, 1};
        if (enc(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)a.w, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    {
        cuuint64_t dims[2] = {a.k, a.rows};
        cuuint64_t strides[1] = {(cuuint64_t)a.k * 2};
        cuuint32_t box[2] = {KS, mt};
        cuuint32_t es[2] = {1, 1};
        if (enc(&ma, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_bf16, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    if (fmt == FMT_Q6K) return launch_one_acc<FMT_Q6K>(mt, a, mw, ma, stream);
    if (fmt == FMT_Q5K) return launch_one_acc<FMT_Q5K>(mt, a, mw, ma, stream);
    return launch_one_acc<FMT_Q4K>(mt, a, mw, ma, stream);
}

cudaError_t launch_qgemm_tc(int fmt, const GemmTcArgs &a, void *a_bf16_scratch, int sm_count, cudaStream_t stream, int *launched) {
    using namespace tc;
    *launched = 0;
    if (a.rows == 0 || a.n == 0) return cudaSuccess;
    *launched = 2;  // the bf16 copy of the activations + the GEMM (+ the split-K sum)
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    const uint32_t mt = a.rows <= 64 ? 64 : (a.rows <= 128 ? 128 : 256);

    {
        const dim3 cgrid((a.k / 8 + 255) / 256, a.rows < 65535u ? a.rows : 65535u);
        const bool vec = a.a_type == ACT_F32 && ((uintptr_t)a.a & 15) == 0 && a.a_off % 4 == 0 && a.a_bs % 4 == 0 && a.a_rs % 4 == 0;
        if (vec) a_to_bf16_kernel<true><<<cgrid, 256, 0, stream>>>(a, (__nv_bfloat16 *)a_bf16_scratch);
        else a_to_bf16_kernel<false><<<cgrid, 256, 0, stream>>>(a, (__nv_bfloat16 *)a_bf16_scratch);
    }
    cudaError_t ce = cudaGetLastError();
    if (ce != cudaSuccess) return ce;

    // CTA pairs: Q4_K, more than 128 rows (256-row activation tiles), at least two 256-row weight tiles
    const bool pair = g_tc_pair > 0 && fmt == FMT_Q4K && a.rows > 128 && a.n >= 4 * TN;
    CUtensorMap mw, ma;
    {   // packed weights as bytes: [n rows][row_bytes], box = one 144-byte block (Q6_K: 224 bytes around one) of 128 rows
        const uint32_t blk_bytes = tc_block_bytes(fmt);
        cuuint64_t dims[2] = {(cuuint64_t)(a.k / QK) * blk_bytes, a.n};
        cuuint64_t strides[1] = {(cuuint64_t)(a.k / QK) * blk_bytes};
        cuuint32_t box[2] = {(cuuint32_t)tc_box_bytes(fmt), TN};
        cuuint32_t es[2] = {1, 1};
        if (strides[0] % 16 != 0) {
            // Q6_K with K not a multiple of 2048: no tensor map for the weights (the kernel copies rows itself)
            std::memset(&mw, 0, sizeof(mw));
        } else if (enc(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)a.w, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
            return cudaErrorInvalidValue;
        }
    }
    {   // bf16 activations [rows][k], box = 64 k (128 bytes, swizzled) x MT rows
        cuuint64_t dims[2] = {a.k, a.rows};
        cuuint64_t strides[1] = {(cuuint64_t)a.k * 2};
        cuuint32_t box[2] = {KS, pair ? 128u : (mt > 256 ? 256u : mt)};
        cuuint32_t es[2] = {1, 1};
        if (enc(&ma, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_bf16_scratch, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    // Too few tiles for the SMs (small n: a tensor-parallel shard, a few prefill rows on a narrow
    // matrix): split K over gridDim.z, partial tiles into the scratch, summed in order by a second kernel.
    const uint32_t ways = splitk_ways(a.rows, a.n, a.k, sm_count);
    if (ways > 1 && !pair) {
        GemmTcArgs b = a;
        b.partial = (float *)((char *)a_bf16_scratch + (((size_t)a.rows * a.k * 2 + 255) & ~(size_t)255));
        cudaError_t e;
        e = fmt == FMT_Q6K ? launch_one_acc<FMT_Q6K>(mt, b, mw, ma, stream, ways)
                           : fmt == FMT_Q5K ? launch_one_acc<FMT_Q5K>(mt, b, mw, ma, stream, ways) : launch_one_acc<FMT_Q4K>(mt, b, mw, ma, stream, ways);
        if (e != cudaSuccess) return e;
        const uint64_t total = (uint64_t)a.rows * a.n;
        const unsigned sgrid = (unsigned)((total + 255) / 256 > (uint64_t)sm_count * 8 ? (uint64_t)sm_count * 8 : (total + 255) / 256);
        splitk_sum_kernel<<<sgrid, 256, 0, stream>>>(b, ways);
        *launched = 3;
        return cudaGetLastError();
    }
    // One or two accumulators per CTA at MT = 256: the 256x256 tile halves the activation traffic
    // but there are half as many tiles; take the shape with the shorter modelled time (waves of
    // tiles over the SMs times the measured cost of a k-step of each shape).
    // 512 activation rows per CTA (all 512 columns of tensor memory for one 128-row weight tile): every
    // dequantized weight feeds twice the tensor-core work of the 256-row tiles. A k-step of such a
    // CTA measured 1.6x the time of a 256-row one, so it pays when it saves more than that in waves
    // of tiles over the SMs. Q6_K only: for Q4_K the two-accumulator 256x256 tile is the better way
    // to the same reuse (it also halves the activation traffic), measured faster in every case.
    if (fmt == FMT_Q5K) return launch_one_acc<FMT_Q5K>(mt, a, mw, ma, stream);  // (one accumulator tile: no wide or tall variants built)
    bool tall = false;
    if (a.rows > 256 && fmt == FMT_Q6K) {
        const uint64_t nt = (a.n + TN - 1) / TN;
        const uint64_t w256 = (nt * ((a.rows + 255) / 256) + sm_count - 1) / sm_count;
        const uint64_t w512 = (nt * ((a.rows + 511) / 512) + sm_count - 1) / sm_count;
        tall = w512 * 16 < w256 * 10;
    }
    if (g_tc_tall >= 0) tall = g_tc_tall != 0 && a.rows > 256;
    if (tall) return fmt == FMT_Q6K ? launch_mt<FMT_Q6K, 512, 1>(a, mw, ma, stream) : launch_mt<FMT_Q4K, 512, 1>(a, mw, ma, stream);
    if (fmt == FMT_Q6K) {  // the larger staged blocks leave room for one accumulator tile only
        switch (mt) {
            case 64: return launch_mt<FMT_Q6K, 64, 1>(a, mw, ma, stream);
            case 128: return launch_mt<FMT_Q6K, 128, 1>(a, mw, ma, stream);
            default: return launch_mt<FMT_Q6K, 256, 1>(a, mw, ma, stream);
        }
    }
    bool wide = a.rows > 128 && a.n >= 2 * TN;
    if (wide) {
        const uint64_t mt_tiles = (a.rows + 255) / 256;
        const uint64_t t1 = ((a.n + TN - 1) / TN) * mt_tiles, t2 = ((a.n + 2 * TN - 1) / (2 * TN)) * mt_tiles;
        const uint64_t w1 = (t1 + sm_count - 1) / sm_count, w2 = (t2 + sm_count - 1) / sm_count;
        wide = w2 * 26 <= w1 * 15;
    }
    if (g_tc_wide >= 0) wide = g_tc_wide != 0;
    if (pair) return launch_mt<FMT_Q4K, 256, 2, true>(a, mw, ma, stream);
    switch (mt) {
        case 64: return launch_mt<FMT_Q4K, 64, 1>(a, mw, ma, stream);
        case 128: return launch_mt<FMT_Q4K, 128, 1>(a, mw, ma, stream);
        default: return wide ? launch_mt<FMT_Q4K, 256, 2>(a, mw, ma, stream) : launch_mt<FMT_Q4K, 256, 1>(a, mw, ma, stream);
    }
}

}  // namespace lb

// Q4_K / Q5_K decode GEMV for 2..8 activation rows on the warp-level int8 tensor-core instruction,
// organised as one stream of equal work shares (arithmetic: see qgemv.cu; the integer dot products
// are the same, only the order of the f32 sums over sub-blocks and k-chunks differs).
//
//  * Unit of work: 16*TILES*WARPS weight rows x one k-chunk (NB = one or two super-blocks per row).
//    The units of all members of the launch, tile after tile, k-chunk after k-chunk, form one
//    sequence; CTA b takes a contiguous span of U/G (or one more) of them, so every CTA streams the
//    same number of bytes whatever the shape (no tail of half-empty waves, no idle SMs on matrices
//    with few rows).
//  * Inside a CTA one producer warp fills a ring of stages: the weights of a unit by ONE tensor-map
//    copy (TMA: a box of rows x 288 or 352 bytes of the packed matrix; rows past the end and the missing
//    half of an odd last k-chunk arrive as zeros) and the int8 activation tiles of the same two
//    super-blocks by one bulk copy, both completing on the stage's mbarrier. Shared memory therefore
//    does not grow with K, and the members of a grouped launch may read different activations.
//  * Each consumer warp owns 16*TILES rows of the tile and keeps their 16x8 accumulators in registers
//    over all k-chunks of its span: no cross-warp reduction, no CTA-wide barrier in the main loop. A
//    warp releases a stage with one mbarrier arrive.
//  * Programmatic dependent launch: weights are requested before the dependency wait. What happens to a finished
//    segment of a tile depends on whether the launch may run ahead of the kernel in front of it:
//    - A dependent launch (its activations come from that kernel) waits before it loads them, so by the time a
//      segment is finished it may write. A span that covers all k-chunks of a tile stores it directly. Otherwise
//      the span that holds the tile's first k-chunk adds up and stores, and the spans behind it hand it their
//      partial 16x8 tiles through a workspace in global memory as {value, flag} pairs (one aligned 8-byte store
//      each, never torn: no fence, no atomic). A contributor's share of such a tile is the first thing it computes
//      and the collector's share the last thing, so the pairs are normally there when they are asked for; the
//      collector's polls are bounded all the same. It sums in span order (= k order) and clears the pairs it took.
//      All CTAs of a launch are resident together (the grid never exceeds the CTAs the SMs hold), so a collector
//      never polls a CTA that cannot run.
//    - A launch that runs ahead (GemvArgs::early: everything it reads is older than the kernel in front) must not
//      write its output before that kernel has completed, and a CTA that waited for that would keep its place on
//      the SM from the next launch. So its CTAs only STAGE: every segment goes to a slot (tile, piece) of a staging
//      region in global memory that belongs to this launch alone, and the CTA leaves (one CTA of the grid waits for
//      the kernel in front before it does, so that the grid's completion still means the completion of everything
//      before it). A second, small kernel launched right behind (qgemv_kq_finalize_kernel) waits for this one,
//      adds the pieces of every tile up in k order and stores them. Nobody polls for a neighbour and the result
//      does not depend on timing. A staging region is claimed with a compare-and-swap on its owner word by the
//      first CTA that gets there and released by the last CTA of the second kernel, so two launches in flight never
//      share one whatever the order in which their CTAs run.
//  * The span of CTA b: the first U mod G spans hold floor(U / G) + 1 units, the others floor(U / G).
//  * Every mbarrier wait is bounded; a wait that gives up sets the host-visible status word.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "kernels.h"
#include "pipe.cuh"
#include "tp_ll.cuh"

namespace lb {
namespace ks {

using namespace pipe;

constexpr int BAR_BYTES = 128;
constexpr int SC_STRIDE = 80;  // decoded scales of one (row, super-block): 16 floats, padded against bank conflicts
constexpr uint32_t PAIR_SPIN_LIMIT = 1u << 20;  // polls of a partial-sum pair before the kernel gives up
constexpr int STAGE_REGIONS = 8;                 // staging regions, taken in rotation by the launches that run ahead
constexpr uint64_t STAGE_BYTES = 6ull << 20;     // partial tiles of one region
constexpr int WORDS_BYTES = 256;                 // control words in front of a region (see the claim in the kernel)

__device__ __forceinline__ uint2 ld_pair(const void *p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

template <int FMT> struct Geo {
    static constexpr int BLK = FMT == FMT_Q5K ? Q5K_BYTES : Q4K_BYTES;
    static constexpr int QS = FMT == FMT_Q5K ? 48 : 16;  // offset of the nibbles inside a block
};

__host__ __device__ constexpr uint32_t act_block_bytes(uint32_t rows) { return 256 * rows + 512; }

// Words of a CTA's trace row (SM clock cycles unless stated)
enum { TR_GT_ENTRY = 0 /* ns */, TR_ENTRY, TR_LOADS_ISSUED, TR_FIRST_DATA, TR_BEFORE_WAIT, TR_AFTER_WAIT, TR_EXIT, TR_GT_EXIT /* ns */,
       TR_SM, TR_UNITS, TR_STARVED, TR_FLAG_SEEN, TR_BARS_READY, TR_FIRST_ISSUED, TR_AFTER_SYNC, TRACE_WORDS = 16 };
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// What a CTA needs before its first copy can start, in one 64-byte line of the parameter space (a new launch finds
// the constant cache cold: every further line the prologue touches costs a miss in series)
struct alignas(64) Head {
    uint32_t rows, nblk, chunks, tiles;  // activation rows; super-blocks per weight row; k-chunks per tile; row tiles of all members
    uint32_t q, rem;                     // units per span: the first `rem` spans hold q + 1, the others q
    uint32_t early, pieces;              // early: bit 0 runs ahead (stages), bit 1 measurement only; pieces: staging slots per tile
    const int8_t *qa0;                   // activation tiles of the first member
    uint2 *pairs;                        // hand-over workspace of dependent launches
    unsigned long long *trace;           // diagnostics, or null
    // ---- second line: read at the end of a segment
    float *stage;                        // staging region of a launch that runs ahead: partial tiles
    uint32_t *words;                     // its control words
    uint32_t launch_id, nfinal;          // owner value; CTAs of the kernel that adds the pieces up
    uint32_t spin;                       // polls before a wait on the staging region gives up
};

template <int NG> struct Maps {
    CUtensorMap m[NG];  // packed weights of each member: [n rows][k/256 * BLK/4 words], box ROWB/4 words x tile rows
};

// NB: super-blocks per k-chunk (1 or 2). MINB: CTAs per SM the register allocation must allow.
template <int FMT, int WARPS, int TILES, int NB, int STAGES, int MINB, int NG>
__global__ void __launch_bounds__((WARPS + 1) * 32, MINB)
qgemv_kq_stream_kernel(const __grid_constant__ Maps<NG> maps, const Head head, GemvGroupT<NG> grp) {
    constexpr int BLK = Geo<FMT>::BLK, ROWB = NB * BLK, QS = Geo<FMT>::QS;
    constexpr int RPW = 16 * TILES;      // rows per consumer warp
    constexpr int RT = RPW * WARPS;      // rows per tile
    constexpr int WBYTES = RT * ROWB;    // weight bytes per stage
    constexpr int EW = 128 * TILES;      // outputs of one warp per tile
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t M = head.rows, nblk = head.nblk, C = head.chunks, early = head.early;
    const uint32_t ABLK = act_block_bytes(M);
    const uint32_t SBYTES = WBYTES + NB * ABLK;
    const uint32_t b = blockIdx.x;
    // Equal shares: the first `rem` spans hold q + 1 units, the others q (q >= 1: the grid never exceeds the units)
    const uint32_t q = head.q, rem = head.rem;
    const uint32_t u_lo = b * q + min(b, rem), u_hi = u_lo + q + (b < rem ? 1u : 0u);
    struct {
        uint2 *pairs;
        unsigned long long *trace;
    } ws = {head.pairs, head.trace};
    const uint32_t G = gridDim.x;
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

    // Timeline of this CTA for the diagnostics call (ws.trace is null unless a trace was asked for): 16 words per CTA
    unsigned long long *trace = ws.trace ? ws.trace + (size_t)b * TRACE_WORDS : nullptr;
    auto stamp = [&](int i) {
        if (trace && lane == 0) trace[i] = (unsigned long long)clock64();
    };
    if (trace && threadIdx.x == 0) {
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        trace[TR_GT_ENTRY] = globaltimer_ns();
        trace[TR_ENTRY] = (unsigned long long)clock64();
        trace[TR_SM] = smid;
        trace[TR_UNITS] = u_hi - u_lo;
    }

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint64_t *full = (uint64_t *)smem, *empty = full + STAGES;
    volatile uint32_t *region_ok = (volatile uint32_t *)(smem + BAR_BYTES - 16);  // 1 once the staging region is this launch's own; 2: the claim gave up
    uint8_t *stages = smem + BAR_BYTES;
    // The producer's lane sets the barriers up and asks for the first weights at once; the others meet it below.
    auto unit = [&](uint32_t i, int &item, uint32_t &local, uint32_t &c, uint32_t &nb) {
        const uint32_t u = u_lo + i, gt = u / C;
        c = u - gt * C;
        item = locate(gt, local);
        nb = min((uint32_t)NB, nblk - NB * c);
    };
    auto load_w = [&](uint32_t i, uint32_t slot) {
        int item;
        uint32_t local, c, nb;
        unit(i, item, local, c, nb);
        mbar_expect_tx(full + slot, WBYTES + nb * ABLK);  // the whole box counts, zero fill included
        tma_load_2d(stages + (size_t)slot * SBYTES, &maps.m[item], (int)(c * (ROWB / 4)), (int)(local * RT), full + slot);
    };
    auto load_a = [&](uint32_t i, uint32_t slot) {
        int item;
        uint32_t local, c, nb;
        unit(i, item, local, c, nb);
        const int8_t *qa = NG == 1 ? head.qa0 : grp.item[item].qa;
        bulk_g2s(stages + (size_t)slot * SBYTES + WBYTES, (const uint8_t *)qa + (size_t)(NB * c) * ABLK, nb * ABLK, full + slot);
    };
    const uint32_t nunits = u_hi - u_lo;
    const uint32_t pre = nunits < (uint32_t)STAGES ? nunits : (uint32_t)STAGES;
    if (warp == WARPS && lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, WARPS);
        }
        *region_ok = 0;
        mbar_fence_init();
        stamp(TR_BARS_READY);
        for (uint32_t i = 0; i < pre; i++) {
            load_w(i, i);
            if (early & 1) load_a(i, i);  // (a launch that runs ahead: its activations are older than the kernel in front)
            if (i == 0) stamp(TR_FIRST_ISSUED);
        }
    }
    __syncthreads();
    if (warp == 0) stamp(TR_AFTER_SYNC);

    if (warp == WARPS) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            if (!(early & 1)) {
                asm volatile("griddepcontrol.wait;" ::: "memory");  // the activations come from the kernel in front
                for (uint32_t i = 0; i < pre; i++) load_a(i, i);
            } else {
                // Claim the staging region: word 0 is its owner (a launch id, 0 = free). Whoever swaps its id into a free
                // word first owns it for the launch; the other CTAs find the id there. The kernel that adds the pieces up
                // frees it. A launch that finds the region owned by an earlier one waits for that (the earlier launch
                // depends on nothing this one does).
                uint32_t ok = 2;
                for (uint32_t spin = 0; spin < head.spin; spin++) {
                    uint32_t o = *(volatile uint32_t *)head.words;
                    if (o == 0) o = atomicCAS(head.words, 0u, head.launch_id) ? *(volatile uint32_t *)head.words : head.launch_id;
                    if (o == head.launch_id) {
                        ok = 1;
                        break;
                    }
                    __nanosleep(64);
                }
                if (ok != 1 && grp.item[0].status) atomicOr(grp.item[0].status, 1);
                *region_ok = ok;
            }
            stamp(TR_LOADS_ISSUED);
            uint32_t slot = 0, phase = 0;  // phase of `empty[slot]` the next refill waits for
            for (uint32_t i = pre; i < nunits; i++) {
                if (!mbar_wait(empty + slot, phase)) {
                    if (grp.item[0].status) atomicOr(grp.item[0].status, 1);
                    break;
                }
                load_w(i, slot);
                load_a(i, slot);
                if (++slot == (uint32_t)STAGES) {
                    slot = 0;
                    phase ^= 1;
                }
            }
        } else {
            // (the idle lanes touch the parameter lines the epilogue reads, so that they are in the constant cache by then)
            const uint32_t touch = grp.item[0].n ^ (uint32_t)(uintptr_t)grp.item[0].out ^ (uint32_t)grp.item[0].out_rs ^ grp.task_end[0] ^
                                   head.launch_id;
            asm volatile("" ::"r"(touch));
        }
        // A launch that runs ahead: one CTA waits for the kernel in front before it leaves, so that this grid's
        // completion still means the completion of everything before it (the others just leave).
        if ((early & 1) && b + 1 == G) asm volatile("griddepcontrol.wait;" ::: "memory");
        return;
    }

    // -------------------------------------------------------------------- consumers
    const int gq = lane >> 2, t4 = lane & 3;
    const uint32_t colq = (uint32_t)gq < M ? gq : 0;      // activation row of this lane's B fragment
    const uint32_t cp = (uint32_t)(2 * t4) < M ? t4 : 0;  // activation row pair of this lane's C fragment
    const uint64_t neg_magic = pack2(-MAGIC, -MAGIC);
    uint8_t *scs = stages + (size_t)STAGES * SBYTES + (size_t)warp * (RPW * NB * SC_STRIDE);  // one slot per (row, super-block) of a stage
    __shared__ TpPushCtx tp_ctx[WARPS];
    bool waited = false, healthy = true;
    auto owner = [&](uint32_t u) -> uint32_t { return u < rem * (q + 1) ? u / (q + 1) : rem + (u - rem * (q + 1)) / q; };

    // Writes a finished tile of member `item` (rows local*RT.. of it), epilogue included.
    auto store = [&](uint32_t gt, uint32_t w, const float (&v)[TILES][4]) {  // w: the warp slice of the tile
        uint32_t local;
        const int item = locate(gt, local);
        const GemvArgs &p = grp.item[item];
#pragma unroll
        for (int tl = 0; tl < TILES; tl++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t row = local * RT + w * RPW + tl * 16 + gq + ((i & 2) ? 8 : 0);
                const uint32_t r = 2 * t4 + (i & 1);
                if (row < p.n && r < M) {
                    float x = v[tl][i];
                    const uint32_t bt = r / p.m, ri = r % p.m;
                    if (p.extra && !p.epi.n) x += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)ri * p.ex_s1 + (int64_t)row * p.ex_s2];
                    if (p.tp) tp_push_value(&tp_ctx[warp], (uint64_t)r * p.n + row, x);  // row-parallel partial: to every rank
                    else p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)ri * p.out_rs + row] = x;
                }
            }
    };
    constexpr int NE = 4 * TILES;  // accumulators of a lane
    // ---- a launch that runs ahead: segment [c0, ..) of tile gt goes to its staging slot (tile, piece); the piece is
    //      the position of this span among the spans that share the tile
    auto stage_out = [&](uint32_t gt, const float (&acc)[TILES][4]) {
        uint32_t ok = *region_ok;
        for (uint32_t spin = 0; spin < PAIR_SPIN_LIMIT && ok == 0; spin++) {  // (the producer's claim is what is bounded by head.spin)
            __nanosleep(32);
            ok = *region_ok;
        }
        if (ok != 1) {
            healthy = false;
            return;
        }
        float *dst = head.stage + (((size_t)gt * head.pieces + (b - owner(gt * C))) * WARPS + warp) * EW + lane;
#pragma unroll
        for (int e = 0; e < NE; e++) __stcg(dst + e * 32, acc[e / 4][e % 4]);
    };
    // ---- a dependent launch. One finished segment [c0, c1) of tile gt: store it, hand it to the span that collects
    //      the tile, or collect.
    auto finish = [&](uint32_t gt, uint32_t c0, uint32_t c1, float (&acc)[TILES][4]) {
        if (!healthy) return;
        if (c0 == 0 && c1 == C) {
            store(gt, warp, acc);
            return;
        }
        if (early & 2) return;  // measurement only (option gemv_stream_debug): partial tiles are dropped, the results are wrong
        // ---- this span holds only some k-chunks of the tile. The span that holds the tile's first k-chunk adds
        //      up and stores; the others hand it their partial sums through the workspace as {value, 1} pairs
        //      (an aligned 8-byte store is never torn, so a pair whose flag is set carries its value: no fence,
        //      no counter). Only the first segment of a span can lack its tile's head, so a CTA has one slot.
        if (c0 != 0) {
            uint2 *mine = ws.pairs + ((size_t)b * WARPS + warp) * EW;
#pragma unroll
            for (int e = 0; e < NE; e++) st_pair(mine + e * 32 + lane, acc[e / 4][e % 4], 1u);
            return;
        }
        // The contributors are the spans right behind this one; theirs is the FIRST thing they compute, so their
        // pairs are usually there already. Sum in span order = k order; take each pair and leave the slot empty
        // for the next launch (which touches the workspace only after this grid has completed).
        const uint32_t b_last = owner(gt * C + C - 1);
        constexpr int NBATCH = 4 / TILES;  // contributors asked for at once (their loads are all in flight together)
        for (uint32_t b0 = b + 1; b0 <= b_last && healthy; b0 += NBATCH) {
            uint2 v[NBATCH][NE];
            auto slot_of = [&](int j, int e) { return ws.pairs + ((size_t)(b0 + j) * WARPS + warp) * EW + e * 32 + lane; };
#pragma unroll
            for (int j = 0; j < NBATCH; j++)
#pragma unroll
                for (int e = 0; e < NE; e++) v[j][e] = b0 + j <= b_last ? ld_pair(slot_of(j, e)) : make_uint2(0u, 1u);
            for (uint32_t spin = 0; spin < PAIR_SPIN_LIMIT; spin++) {
                bool all = true;
#pragma unroll
                for (int j = 0; j < NBATCH; j++)
#pragma unroll
                    for (int e = 0; e < NE; e++) all = all && v[j][e].y != 0;
                if (all) break;
#pragma unroll
                for (int j = 0; j < NBATCH; j++)
#pragma unroll
                    for (int e = 0; e < NE; e++)
                        if (v[j][e].y == 0) v[j][e] = ld_pair(slot_of(j, e));
            }
#pragma unroll
            for (int j = 0; j < NBATCH; j++)
#pragma unroll
                for (int e = 0; e < NE; e++) {
                    if (v[j][e].y == 0) healthy = false;
                    if (b0 + j <= b_last) {
                        acc[e / 4][e % 4] += __uint_as_float(v[j][e].x);
                        st_pair(slot_of(j, e), 0.0f, 0u);
                    }
                }
        }
        healthy = __all_sync(0xffffffffu, healthy);
        if (!healthy) {
            if (lane == 0 && grp.item[0].status) atomicOr(grp.item[0].status, 1);
            return;
        }
        store(gt, warp, acc);
    };

    uint32_t u = u_lo, slot = 0, par = 0;
    long long starved = 0;  // (trace) cycles warp 0 waited for data
    while (u < u_hi) {
        const uint32_t gt = u / C, c0 = u - gt * C;
        const uint32_t c1 = min(C, c0 + (u_hi - u));
        float acc[TILES][4];
#pragma unroll
        for (int tl = 0; tl < TILES; tl++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[tl][i] = 0.0f;

        for (uint32_t c = c0; c < c1; c++, u++) {
            const long long t_wait = trace ? clock64() : 0;
            if (healthy && !mbar_wait(full + slot, par)) {
                healthy = false;
                if (lane == 0 && grp.item[0].status) atomicOr(grp.item[0].status, 1);
            }
            if (trace && warp == 0) {
                starved += clock64() - t_wait;
                if (u == u_lo) stamp(TR_FIRST_DATA);
            }
            const uint8_t *wst = stages + (size_t)slot * SBYTES + (size_t)warp * (RPW * ROWB);  // this warp's rows
            const uint8_t *ast = stages + (size_t)slot * SBYTES + WBYTES;
            const uint32_t nb = min((uint32_t)NB, nblk - NB * c);
            if (healthy) {
                // ---- decode the 6-bit scales and mins: one lane per (row, super-block); per sub-block pair j
                //      {d*sc[2j], d*sc[2j+1] (/16 where the high nibbles are used in place), -dmin*m[2j], -dmin*m[2j+1]}
                auto decode = [&](uint32_t rr, uint32_t bb, uint32_t sl) {
                    const uint4 h = *(const uint4 *)(wst + rr * ROWB + bb * BLK);
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
                        w[s] = (FMT == FMT_Q4K && (s & 1)) ? sc * 0.0625f : sc;
                        w[8 + s] = scale_byte(s < 4 ? mn_lo : mn_hi, sel, dmin, ndmin);
                    }
                    float4 *dst = (float4 *)(scs + sl * SC_STRIDE);
#pragma unroll
                    for (int j = 0; j < 4; j++) dst[j] = make_float4(w[2 * j], w[2 * j + 1], w[8 + 2 * j], w[8 + 2 * j + 1]);
                };
                if constexpr (TILES == 2) {  // a lane per row, one super-block after the other
#pragma unroll
                    for (uint32_t bb = 0; bb < (uint32_t)NB; bb++)
                        if (bb < nb) decode(lane, bb, bb * RPW + lane);
                } else if constexpr (NB == 2) {  // 16 rows x 2 super-blocks
                    if ((uint32_t)(lane >> 4) < nb) decode(lane & 15, lane >> 4, lane);
                } else {
                    if (lane < 16) decode(lane, 0, lane);
                }
                __syncwarp();
#pragma unroll
                for (uint32_t bb = 0; bb < (uint32_t)NB; bb++) {
                    if (bb >= nb) break;
                    const uint8_t *ab = ast + (size_t)bb * ABLK;
                    const float4 *dsp = (const float4 *)(ab + 256 * M) + cp;  // scales: [sub-block pair][row pair][sub-block & 1][row & 1]
                    ulonglong2 dav[4];  // {da[c0], da[c1]} of sub-blocks 2i, 2i + 1
                    float4 bsv[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        dav[i] = ((const ulonglong2 *)dsp)[4 * i];
                        bsv[i] = dsp[16 + 4 * i];
                    }
                    const float *bs = (const float *)bsv;  // [sub-block][2]
                    uint2 qh[TILES][2];                    // Q5_K: the fifth bits of this lane's eight k positions, rows gq and gq + 8
                    if constexpr (FMT == FMT_Q5K) {
#pragma unroll
                        for (int tl = 0; tl < TILES; tl++)
#pragma unroll
                            for (int hf = 0; hf < 2; hf++)
                                qh[tl][hf] = *(const uint2 *)(wst + (tl * 16 + hf * 8 + gq) * ROWB + bb * BLK + 16 + 8 * t4);
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const uint2 blo = *(const uint2 *)(ab + (2 * j) * (M * 32) + colq * 32 + 8 * t4);
                        const uint2 bhi = *(const uint2 *)(ab + (2 * j + 1) * (M * 32) + colq * 32 + 8 * t4);
#pragma unroll
                        for (int tl = 0; tl < TILES; tl++) {
                            const uint8_t *wrow = wst + (tl * 16 + gq) * ROWB + bb * BLK + QS + j * 32 + 8 * t4;
                            const uint2 wa = *(const uint2 *)wrow, wb = *(const uint2 *)(wrow + 8 * ROWB);
                            uint32_t al[4], ah[4];
                            if constexpr (FMT == FMT_Q5K) {
                                // bit 2j (2j + 1) of a qh byte is the fifth bit of the low (high) nibble's weight
                                auto fifth = [](uint32_t q, int bit) { return (bit <= 4 ? q << (4 - bit) : q >> (bit - 4)) & 0x10101010u; };
                                al[0] = (wa.x & 0x0F0F0F0Fu) | fifth(qh[tl][0].x, 2 * j);
                                al[1] = (wb.x & 0x0F0F0F0Fu) | fifth(qh[tl][1].x, 2 * j);
                                al[2] = (wa.y & 0x0F0F0F0Fu) | fifth(qh[tl][0].y, 2 * j);
                                al[3] = (wb.y & 0x0F0F0F0Fu) | fifth(qh[tl][1].y, 2 * j);
                                ah[0] = ((wa.x >> 4) & 0x0F0F0F0Fu) | fifth(qh[tl][0].x, 2 * j + 1);
                                ah[1] = ((wb.x >> 4) & 0x0F0F0F0Fu) | fifth(qh[tl][1].x, 2 * j + 1);
                                ah[2] = ((wa.y >> 4) & 0x0F0F0F0Fu) | fifth(qh[tl][0].y, 2 * j + 1);
                                ah[3] = ((wb.y >> 4) & 0x0F0F0F0Fu) | fifth(qh[tl][1].y, 2 * j + 1);
                            } else {
                                al[0] = wa.x & 0x0F0F0F0Fu, al[1] = wb.x & 0x0F0F0F0Fu, al[2] = wa.y & 0x0F0F0F0Fu, al[3] = wb.y & 0x0F0F0F0Fu;
                                ah[0] = wa.x & 0xF0F0F0F0u, ah[1] = wb.x & 0xF0F0F0F0u, ah[2] = wa.y & 0xF0F0F0F0u, ah[3] = wb.y & 0xF0F0F0F0u;
                            }
                            int cl[4], ch[4];
                            mma_u8s8_magic(cl, al[0], al[1], al[2], al[3], blo.x, blo.y);
                            mma_u8s8_magic(ch, ah[0], ah[1], ah[2], ah[3], bhi.x, bhi.y);
                            // int -> f32 and the activation scale on packed f32x2: the two outputs of a
                            // row are one register pair, and so are their activation scales
                            float gl[4], gh[4];
                            unpack2(mul2(add2(pack2i(cl[0], cl[1]), neg_magic), dav[j].x), gl[0], gl[1]);
                            unpack2(mul2(add2(pack2i(cl[2], cl[3]), neg_magic), dav[j].x), gl[2], gl[3]);
                            unpack2(mul2(add2(pack2i(ch[0], ch[1]), neg_magic), dav[j].y), gh[0], gh[1]);
                            unpack2(mul2(add2(pack2i(ch[2], ch[3]), neg_magic), dav[j].y), gh[2], gh[3]);
                            const uint32_t sl = bb * RPW + tl * 16 + gq;
                            const float4 sv0 = ((const float4 *)(scs + sl * SC_STRIDE))[j];
                            const float4 sv1 = ((const float4 *)(scs + (sl + 8) * SC_STRIDE))[j];
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                const float4 sv = (i & 2) ? sv1 : sv0;
                                const int cc = i & 1;
                                float a = acc[tl][i];
                                a = fmaf(gl[i], sv.x, a);
                                a = fmaf(sv.z, bs[(2 * j) * 2 + cc], a);
                                a = fmaf(gh[i], sv.y, a);
                                a = fmaf(sv.w, bs[(2 * j + 1) * 2 + cc], a);
                                acc[tl][i] = a;
                            }
                        }
                    }
                }
            }
            __syncwarp();  // every lane is done with the stage and the scale scratch
            if (lane == 0) mbar_arrive(empty + slot);
            if (++slot == (uint32_t)STAGES) {
                slot = 0;
                par ^= 1;
            }
        }

        if (u >= u_hi && warp == 0) stamp(TR_BEFORE_WAIT);
        if (early & 1) {  // runs ahead: nothing is written but the staging region
            if (healthy) stage_out(gt, acc);
            continue;
        }
        if (!waited) {  // (the producer has waited already before it asked for the activations: this returns at once)
            asm volatile("griddepcontrol.wait;" ::: "memory");
            waited = true;
            if (warp == 0) stamp(TR_AFTER_WAIT);
            if (grp.item[0].tp) {  // only the first member of a launch may push (tensor-parallel launches are never grouped)
                if (lane == 0) tp_push_ctx_load(&tp_ctx[warp], grp.item[0].tp);
                __syncwarp();
            }
        }
        finish(gt, c0, c1, acc);
    }
    if (trace && warp == 0 && lane == 0) {
        trace[TR_STARVED] = (unsigned long long)starved;
        trace[TR_EXIT] = (unsigned long long)clock64();
        trace[TR_GT_EXIT] = globaltimer_ns();
    }
}

// Second half of a launch that ran ahead: adds the staged pieces of every (tile, warp slice) up in k order and stores
// the result (epilogue included). Launched right behind the stream kernel, it waits for that kernel -- and through its
// one waiting CTA for everything before it -- so the pieces are complete and the output may be written; the stream
// kernel's CTAs meanwhile have left their SMs to the next launch. One item per warp and round, all its pieces in flight
// together. The last CTA frees the staging region.
// EXPR: a member has an epilogue expression (a variant of its own: the evaluator's code and stack stay out of the other).
template <int WARPS, int TILES, int NG, bool EXPR>
__global__ void __launch_bounds__(256) qgemv_kq_finalize_kernel(const Head head, GemvGroupT<NG> grp) {
    constexpr int RPW = 16 * TILES, RT = RPW * WARPS, EW = 128 * TILES, NE = 4 * TILES;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = threadIdx.x & 31, gq = lane >> 2, t4 = lane & 3;
    const uint32_t C = head.chunks, q = head.q, rem = head.rem, M = head.rows;
    auto owner = [&](uint32_t u) -> uint32_t { return u < rem * (q + 1) ? u / (q + 1) : rem + (u - rem * (q + 1)) / q; };
    // (what the loop needs of the parameters, fetched before the wait)
    const uint32_t items = head.tiles * WARPS, wpc = blockDim.x >> 5;
    const uint32_t touch = grp.item[0].n ^ (uint32_t)(uintptr_t)grp.item[0].out ^ grp.task_end[0];
    asm volatile("" ::"r"(touch));
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t it = blockIdx.x * wpc + (threadIdx.x >> 5); it < items; it += gridDim.x * wpc) {
        const uint32_t t = it / WARPS, w = it - t * WARPS;
        const uint32_t np = owner(t * C + C - 1) - owner(t * C) + 1;
        const float *src = head.stage + (((size_t)t * head.pieces) * WARPS + w) * EW + lane;
        float acc[NE];
#pragma unroll
        for (int e = 0; e < NE; e++) acc[e] = 0.0f;
        for (uint32_t p0 = 0; p0 < np; p0 += 4) {
            float v[4][NE];
#pragma unroll
            for (int j = 0; j < 4; j++)
#pragma unroll
                for (int e = 0; e < NE; e++) v[j][e] = p0 + j < np ? __ldcg(src + (size_t)(p0 + j) * WARPS * EW + e * 32) : 0.0f;
#pragma unroll
            for (int j = 0; j < 4; j++)
#pragma unroll
                for (int e = 0; e < NE; e++) acc[e] += v[j][e];
        }
        uint32_t local = t;
        int item = 0;
        if constexpr (NG > 1) {
            while (t >= grp.task_end[item]) item++;
            local = t - (item ? grp.task_end[item - 1] : 0);
        }
        const GemvArgs &p = grp.item[item];
#pragma unroll
        for (int e = 0; e < NE; e++) {
            const int tl = e / 4, i = e % 4;
            const uint32_t row = local * RT + w * RPW + tl * 16 + gq + ((i & 2) ? 8 : 0);
            const uint32_t r = 2 * t4 + (i & 1);
            if (row < p.n && r < M) {
                float x = acc[e];
                const uint32_t bt = r / p.m, ri = r % p.m;
                const int64_t ex = (int64_t)(p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)ri * p.ex_s1 + (int64_t)row * p.ex_s2);
                if constexpr (EXPR) x = epilogue(p, x, ex);
                else if (p.extra) x += p.extra[ex];
                p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)ri * p.out_rs + row] = x;
            }
        }
    }
    // the last CTA to get here frees the staging region (every read of it lies before that CTA's count)
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(head.words + 2, 1u) == gridDim.x - 1) {
        head.words[2] = 0;
        __threadfence();
        *(volatile uint32_t *)head.words = 0;
    }
}

// ------------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static std::mutex g_mu;  // guards the caches below: launches may come from several host threads (one per device)

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!tried) {
        tried = true;
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// A tensor map depends only on (address, n, k, block bytes, box rows): the last few are remembered, a
// decode loop asks for the same handful every token.
static bool weight_map(const GemvArgs &a, uint32_t blk, uint32_t nb, uint32_t box_rows, CUtensorMap &out) {
    struct Entry {
        const void *w;
        uint32_t n, k, blk, nb, rows;
        CUtensorMap map;
    };
    constexpr int CAP = 256;
    static Entry cache[CAP];
    static int used = 0, next = 0;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    std::lock_guard<std::mutex> lock(g_mu);
    for (int i = 0; i < used; i++)
        if (cache[i].w == a.w && cache[i].n == a.n && cache[i].k == a.k && cache[i].blk == blk && cache[i].nb == nb && cache[i].rows == box_rows) {
            out = cache[i].map;
            return true;
        }
    const uint32_t nblk = a.k / QK;
    cuuint64_t dims[2] = {(cuuint64_t)nblk * (blk / 4), a.n};
    cuuint64_t strides[1] = {(cuuint64_t)nblk * blk};
    cuuint32_t box[2] = {nb * blk / 4, box_rows};
    cuuint32_t es[2] = {1, 1};
    if (enc(&out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void *)a.w, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    Entry &e = cache[used < CAP ? used++ : (next = (next + 1) % CAP)];
    e.w = a.w;
    e.n = a.n;
    e.k = a.k;
    e.blk = blk;
    e.nb = nb;
    e.rows = box_rows;
    e.map = out;
    return true;
}

// Layouts (consumer warps, 16-row tiles per warp, super-blocks per k-chunk, ring stages):
// 0: eight warps of 16 rows, two-block chunks, two stages
// 1: four warps of 32 rows (the activation fragments and scales are shared by two row tiles), two-block chunks, two stages
// 2: four warps of 16 rows, two-block chunks, three stages
// 3: four warps of 16 rows, two-block chunks, two stages (three CTAs per SM): the default up to 66 MB
// 4: three warps of 16 rows, two-block chunks, two stages (four CTAs per SM)
// (Also built and measured, never ahead: one-block chunks with three and four stages, eight warps of 32 rows, six and
// two warps of 16 rows.)
constexpr int N_CONFIGS = 5;
static int g_force_config = -1;
static int g_ctas_per_sm = 0;  // 0 = choose
static int g_debug = 0;        // bits: 2 = drop the partial tiles (measurement only: wrong results); 4 = no launch runs ahead;
                               // 8 = test hook, see launch_n
// Tuning: CTAs per SM of a launch that runs ahead of its predecessor (0 = as pick_config says).
static int g_early_ctas = 0;
static int g_spin_limit = 0;   // polls before the claim of a staging region gives up (0 = PAIR_SPIN_LIMIT); tests shorten it
static int g_big_units = 16;   // tuning: 128-row units per SM from which the 32-row warps are used
static int g_final_tiles = 0;  // tuning: row tiles per finalising CTA of a launch that runs ahead (0 = choose)
// Diagnostics: a device buffer of TRACE_WORDS words per CTA for the next `g_trace_cap` launches (row = launch, in launch order)
static unsigned long long *g_trace = nullptr;
static uint32_t g_trace_cap = 0, g_trace_next = 0, g_trace_ctas = 0;

static size_t smem_bytes(int fmt, int warps, int tiles, int nb, int stages, uint32_t rows) {
    const size_t rowb = (size_t)nb * (fmt == FMT_Q5K ? Geo<FMT_Q5K>::BLK : Geo<FMT_Q4K>::BLK);
    const size_t stage = (size_t)16 * tiles * warps * rowb + nb * act_block_bytes(rows);
    return BAR_BYTES + (size_t)stages * stage + (size_t)warps * 16 * tiles * nb * SC_STRIDE;
}

template <int FMT, int WARPS, int TILES, int NB, int STAGES, int MINB, int NG>
static cudaError_t launch_n(GemvGroupT<NG> &g, StreamWs &ws, int sm_count, bool pdl, bool early, int want_per_sm, cudaStream_t stream) {  // NOLINT
    auto kern = qgemv_kq_stream_kernel<FMT, WARPS, TILES, NB, STAGES, MINB, NG>;
    constexpr uint32_t RT = 16 * TILES * WARPS;
    const uint32_t M = g.item[0].rows, C = (g.item[0].k / QK + NB - 1) / NB;
    uint32_t tiles = 0;
    Maps<NG> maps;
    for (int i = 0; i < g.count; i++) {
        tiles += (g.item[i].n + RT - 1) / RT;
        g.task_end[i] = tiles;
        if (!weight_map(g.item[i], Geo<FMT>::BLK, NB, RT, maps.m[i])) return cudaErrorNotSupported;
    }
    for (int i = g.count; i < NG; i++) maps.m[i] = maps.m[0];
    const size_t smem = smem_bytes(FMT, WARPS, TILES, NB, STAGES, M);
    static DynamicSmemOptIn opted;
    if (cudaError_t e = opted.raise((const void *)kern, smem); e != cudaSuccess) return e;
    // As many CTAs per SM as fit, at most what the kernel's register allocation allows (measured: a CTA slot left to
    // the next launch of the stream costs more than it brings here). The grid never exceeds what the SMs hold at
    // once: see the kernel's hand-over.
    const uint32_t fit = (uint32_t)((227 * 1024) / (smem + 1024));
    uint32_t per_sm = fit < (uint32_t)MINB ? (fit ? fit : 1) : (uint32_t)MINB;
    // Tuning: a launch that runs ahead of its predecessor may leave CTA slots to the launches around it.
    if (early && fit >= 2 && g_early_ctas > 0) per_sm = (uint32_t)g_early_ctas < per_sm ? (uint32_t)g_early_ctas : per_sm;
    if (want_per_sm > 0) per_sm = (uint32_t)want_per_sm < per_sm ? (uint32_t)want_per_sm : per_sm;
    if (g_ctas_per_sm > 0) per_sm = (uint32_t)g_ctas_per_sm < per_sm ? (uint32_t)g_ctas_per_sm : per_sm;
    const uint64_t U = (uint64_t)tiles * C;
    if (U >= (1ull << 31)) return cudaErrorNotSupported;
    uint32_t grid = (uint32_t)sm_count * per_sm;
    if (grid > U) grid = (uint32_t)U;
    // workspace: one partial tile (RT x 8 pairs) per CTA
    if ((uint64_t)grid * RT * 8 > ws.n_pairs || !ws.pairs) return cudaErrorNotSupported;
    // A launch that runs ahead stages its segments: at most `pieces` spans share a tile. Without room for that it runs
    // as a dependent launch.
    const uint32_t q = (uint32_t)(U / grid), pieces = (C + q - 1) / q + 1;
    if (early && ((uint64_t)tiles * pieces * RT * 8 * 4 > STAGE_BYTES || !ws.stage || (g_debug & 4))) {
        early = false;
        for (int i = 0; i < g.count; i++) g.item[i].early = 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3((WARPS + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    Head head = {};
    head.rows = M;
    head.nblk = g.item[0].k / QK;
    head.chunks = C;
    head.tiles = tiles;
    head.q = q;
    head.rem = (uint32_t)(U % grid);
    head.early = (uint32_t)((early ? 1 : 0) | (g_debug & 2));
    head.pieces = pieces;
    head.qa0 = g.item[0].qa;
    head.pairs = ws.pairs;
    if (early) {
        uint8_t *region = ws.stage + (size_t)(ws.next_region++ % STAGE_REGIONS) * (WORDS_BYTES + STAGE_BYTES);
        head.words = (uint32_t *)region;
        head.stage = (float *)(region + WORDS_BYTES);
        if (++ws.next_id == 0) ws.next_id = 1;
        head.launch_id = ws.next_id;
        head.spin = g_spin_limit > 0 ? (uint32_t)g_spin_limit : PAIR_SPIN_LIMIT;
        if (g_debug & 8) {  // test hook: the region looks owned by a launch that never frees it, so the claim runs out
            static const uint32_t foreign = 0x7FFFFFFFu;
            if (cudaError_t e = cudaMemcpyAsync(head.words, &foreign, 4, cudaMemcpyHostToDevice, stream); e != cudaSuccess) return e;
        }
        const uint32_t per = g_final_tiles > 0 ? (uint32_t)g_final_tiles : 16;  // items (tile x warp slice) per CTA of the adding-up kernel
        head.nfinal = (tiles * WARPS + per - 1) / per;
    }
    if (g_trace && g_trace_next < g_trace_cap && grid <= g_trace_ctas)
        head.trace = g_trace + (size_t)(g_trace_next++) * g_trace_ctas * TRACE_WORDS;
    ws.kernels += early ? 2 : 1;
    if (cudaError_t e = cudaLaunchKernelEx(&cfg, kern, maps, head, g); e != cudaSuccess || !early) return e;
    // the launch ran ahead: its second half (see qgemv_kq_finalize_kernel)
    cudaLaunchConfig_t fin = {};
    fin.gridDim = dim3(head.nfinal);
    fin.blockDim = dim3(256);
    fin.stream = stream;
    fin.attrs = attr;
    fin.numAttrs = 1;
    bool expr = false;
    for (int i = 0; i < g.count; i++) expr = expr || g.item[i].epi.n != 0;
    const cudaError_t e = expr ? cudaLaunchKernelEx(&fin, qgemv_kq_finalize_kernel<WARPS, TILES, NG, true>, head, g)
                               : cudaLaunchKernelEx(&fin, qgemv_kq_finalize_kernel<WARPS, TILES, NG, false>, head, g);
    for (int i = 0; i < g.count; i++) g.item[i].epi.n = 0;  // (the adding-up kernel has evaluated the members' expressions)
    return e;
}

template <int FMT, int WARPS, int TILES, int NB, int STAGES, int MINB>
static cudaError_t launch_cfg(GemvGroup &g, StreamWs &ws, int sm_count, bool pdl, bool early, int per_sm, cudaStream_t stream) {
    if (g.count > 1) return launch_n<FMT, WARPS, TILES, NB, STAGES, MINB, GEMV_GROUP_MAX>(g, ws, sm_count, pdl, early, per_sm, stream);
    GemvSingle one;  // a lone launch passes a sixth of the parameter bytes
    one.item[0] = g.item[0];
    one.act_off[0] = 0;
    one.act_copy[0] = 0;
    one.count = 1;
    one.act_bytes = 0;
    const cudaError_t e = launch_n<FMT, WARPS, TILES, NB, STAGES, MINB, 1>(one, ws, sm_count, pdl, early, per_sm, stream);
    g.item[0].epi.n = one.item[0].epi.n;  // (cleared when the launch evaluated its expression itself)
    g.item[0].early = one.item[0].early;
    return e;
}

// Measured (M = 4, 8; early = launches that run ahead of their predecessor, as in a list over one quantized operand):
//  * four warps of 16 rows, two-block chunks, two stages (57 KB: three CTAs fit on an SM) up to 66 MB; what counts at
//    these sizes is that the SM is never without a CTA that computes while another starts or hands over, so three
//    CTAs per SM -- or two with the third slot left to the next launch of the stream when the spans would
//    otherwise fall below six units (many spans per row tile: more hand-overs than work);
//  * below two units per SM (4096 x 4096 at Q5_K: 4.8 against 6.6 us) one CTA of three stages per SM;
//  * from sixteen 128-row units per SM on the 32-row warps, whose activation fragments and scales serve two row tiles
//    (shared-memory wavefronts bound the 16-row layout in the long run).
static int pick_config(const GemvGroup &g, int sm_count, bool early, int &per_sm) {
    per_sm = 0;
    if (g_force_config >= 0) return g_force_config;
    uint64_t units = 0;  // 128 rows x 512 k
    for (int i = 0; i < g.count; i++) units += (uint64_t)((g.item[i].n + 127) / 128) * ((g.item[i].k / QK + 1) / 2);
    if (units >= (uint64_t)g_big_units * (uint64_t)sm_count) return 1;
    if (units < 2 * (uint64_t)sm_count) {  // small matrices (Q5_K only: Q4_K has the per-warp-ring kernel for them): one CTA of three stages per SM
        per_sm = 1;
        return 2;
    }
    if (early && 2 * units < 6 * 3 * (uint64_t)sm_count) per_sm = 2;  // (64-row tiles: twice the units)
    return 3;
}

template <int FMT> static cudaError_t launch_fmt(GemvGroup &g, StreamWs &ws, int sm_count, bool pdl, bool early, cudaStream_t stream) {
    int per_sm = 0;
    switch (pick_config(g, sm_count, early, per_sm)) {
        case 0: return launch_cfg<FMT, 8, 1, 2, 2, 2>(g, ws, sm_count, pdl, early, per_sm, stream);
        case 1: return launch_cfg<FMT, 4, 2, 2, 2, 2>(g, ws, sm_count, pdl, early, per_sm, stream);
        case 2: return launch_cfg<FMT, 4, 1, 2, 3, 2>(g, ws, sm_count, pdl, early, per_sm, stream);
        case 3: return launch_cfg<FMT, 4, 1, 2, 2, 3>(g, ws, sm_count, pdl, early, per_sm, stream);
        case 4: return launch_cfg<FMT, 3, 1, 2, 2, 4>(g, ws, sm_count, pdl, early, per_sm, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ks

void qgemv_kq_stream_set_config(int index) { ks::g_force_config = index < 0 || index >= ks::N_CONFIGS ? -1 : index; }
void qgemv_kq_stream_set_ctas_per_sm(int n) { ks::g_ctas_per_sm = n < 0 ? 0 : n; }
void qgemv_kq_stream_set_debug(int v) { ks::g_debug = v; }
void qgemv_kq_stream_set_early_ctas(int v) { ks::g_early_ctas = v < 0 ? 0 : v; }
void qgemv_kq_stream_set_final_tiles(int v) { ks::g_final_tiles = v < 0 ? 0 : v; }
void qgemv_kq_stream_set_big_units(int v) { ks::g_big_units = v < 1 ? 16 : v; }
void qgemv_kq_stream_set_spin_limit(int v) { ks::g_spin_limit = v < 0 ? 0 : v; }

// Diagnostics: record the timeline of every CTA of the next `launches` launches of this kernel (0 = stop and free).
cudaError_t qgemv_kq_stream_trace_begin(uint32_t launches, int sm_count) {
    if (ks::g_trace) cudaFree(ks::g_trace);
    ks::g_trace = nullptr;
    ks::g_trace_cap = ks::g_trace_next = 0;
    if (!launches) return cudaSuccess;
    ks::g_trace_ctas = (uint32_t)sm_count * 8;
    const size_t bytes = (size_t)launches * ks::g_trace_ctas * ks::TRACE_WORDS * 8;
    if (cudaError_t e = cudaMalloc(&ks::g_trace, bytes); e != cudaSuccess) return e;
    ks::g_trace_cap = launches;
    return cudaMemset(ks::g_trace, 0, bytes);
}
// Copies the rows recorded so far to `out` (launches x ctas x 16 words); returns the launches recorded.
uint32_t qgemv_kq_stream_trace_read(unsigned long long *out, uint64_t cap_words, uint32_t *ctas) {
    if (ctas) *ctas = ks::g_trace_ctas;
    if (!ks::g_trace) return 0;
    uint64_t words = (uint64_t)ks::g_trace_next * ks::g_trace_ctas * ks::TRACE_WORDS;
    if (words > cap_words) words = cap_words;
    if (out && words) cudaMemcpy(out, ks::g_trace, words * 8, cudaMemcpyDeviceToHost);
    return ks::g_trace_next;
}

size_t qgemv_kq_stream_ws_bytes(int sm_count, StreamWs *layout) {
    const uint64_t n_pairs = (uint64_t)sm_count * 4 * 128 * 8;  // up to 4 CTAs per SM of 128-row tiles (or 8 of 64-row ones)
    const uint64_t total = n_pairs * 8 + (uint64_t)ks::STAGE_REGIONS * (ks::WORDS_BYTES + ks::STAGE_BYTES);
    if (layout) {
        layout->n_pairs = n_pairs;
        layout->total_bytes = total;
    }
    return total;
}

bool qgemv_kq_stream_shape_ok(int fmt, uint32_t rows, uint32_t n, uint32_t k) {
    (void)n;
    if (fmt != FMT_Q4K && fmt != FMT_Q5K) return false;
    return rows >= 1 && rows <= 8 && k % QK == 0 && k >= QK && ks::encode_fn() != nullptr;
}

cudaError_t launch_qgemv_kq_stream(int fmt, GemvGroup &g, StreamWs &ws, int sm_count, bool pdl, cudaStream_t stream) {
    if (g.count < 1 || g.count > GEMV_GROUP_MAX) return cudaErrorInvalidValue;
    bool early = pdl;  // every member early and no tensor-parallel push
    for (int i = 0; i < g.count; i++) early = early && g.item[i].early != 0 && g.item[i].tp == nullptr;
    return fmt == FMT_Q5K ? ks::launch_fmt<FMT_Q5K>(g, ws, sm_count, pdl, early, stream)
                          : ks::launch_fmt<FMT_Q4K>(g, ws, sm_count, pdl, early, stream);
}

}  // namespace lb

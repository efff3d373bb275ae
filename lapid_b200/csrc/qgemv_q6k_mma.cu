// Q6_K decode GEMV for 2..8 activation rows on the warp-level int8 tensor-core instruction; the
// Q6_K sibling of qgemv_q4k_mma.cu (same CTA structure: warps split K, per-warp TMA rings,
// activations as tiles in shared memory, partial tiles summed in warp order). Arithmetic as in
// qgemv.cu: exact integer dot products per 16 weights, the int8 sub-scale applied in integers,
// one f32 step per 32-element activation group (crates/lapid-cpu/src/kquant.rs:202-244).
//
// What differs from Q4_K:
//  * A super-block is ql[128] | qh[64] | int8 sc[16] | f16 d = 210 bytes: it starts on a 2-byte
//    boundary only. The tensor-map copy of a stage starts at the 16-byte boundary below the block
//    and takes 224 bytes per row (zero fill past the end of the row); all shared-memory reads of
//    packed bytes are 16-bit loads.
//  * Scales change every 16 weights, so the instruction is `mma.sync.m16n8k16.s8.s8` (16 weight
//    rows x 16 k x 8 activation rows), two per 32-element activation group; their results are
//    combined in integers, sc0 * dot0 + sc1 * dot1, before the one int -> f32 step of the group.
//  * The 6-bit weight q in 0..63 stands for q - 32. (q ^ 32) is its 6-bit two's complement, so the
//    byte ((q ^ 32) << 2) is the int8 value 4 * (q - 32): the low nibble goes to bits 2..5, the two
//    high bits to bits 6..7 with the top one flipped, and the exact factor 1/4 goes into d. Four
//    logic operations per register of four weights.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "kernels.h"
#include "tp_ll.cuh"

namespace lb {
namespace m6 {

constexpr int STAGES = 2;
constexpr int BOX = 224;  // bytes staged per row and super-block
constexpr int BAR_BYTES = 256;

__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
// x counts bytes of a row of the packed matrix (a multiple of 16), y rows
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

// 16 weight rows x 16 k x 8 activation rows, signed bytes, fresh accumulators
__device__ __forceinline__ void mma_s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// a 32-bit word at a 2-byte aligned shared address
__device__ __forceinline__ uint32_t lds_u32_align2(const uint8_t *p) {
    const uint16_t *h = (const uint16_t *)p;
    return (uint32_t)h[0] | ((uint32_t)h[1] << 16);
}
// byte `i` of w, sign-extended (one PRMT: selector 8 | i replicates the byte's sign bit)
__device__ __forceinline__ int sbyte(uint32_t w, int i) {
    int r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0u), "r"(((8u | i) << 12) | ((8u | i) << 8) | ((8u | i) << 4) | (uint32_t)i));
    return r;
}

__host__ __device__ constexpr uint32_t act_block_bytes(uint32_t rows) { return 256 * rows + 512; }  // as the Q4_K kernel's tiles

template <int NG> struct WeightMapsT {
    CUtensorMap m[NG];  // packed weights of each member as bytes: [n rows][k/256 * 210], box 224 x 16*TILES rows
};

template <int WARPS, int TILES, int NG>
__global__ void __launch_bounds__(WARPS * 32, 1)
qgemv_q6k_mma_kernel(const __grid_constant__ WeightMapsT<NG> maps, GemvGroupT<NG> grp) {
    constexpr int THREADS = WARPS * 32;
    constexpr int RPT = 16 * TILES;    // weight rows per tile
    constexpr int STAGE = RPT * BOX;   // bytes per ring stage: one super-block of every row of the tile
    constexpr int ELEMS = RPT * 8;     // outputs per tile
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gq = lane >> 2, t4 = lane & 3;
    const uint32_t M = grp.item[0].rows;
    const uint32_t nblk = grp.item[0].k / QK;  // k-chunks per tile = super-blocks; warp w takes w, w + WARPS, ...
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
    float *red = (float *)(smem + BAR_BYTES + (size_t)WARPS * STAGES * STAGE);  // [2][WARPS][ELEMS]
    uint8_t *acts = (uint8_t *)(red + 2 * WARPS * ELEMS);

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) mbar_init(bars + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    uint32_t pt = t_lo, pit = warp, pslot = 0;
    auto issue = [&]() {
        if (pt >= t_hi || (uint32_t)warp >= nblk) return;
        if (lane == 0) {
            uint32_t local;
            const int item = locate(pt, local);
            mbar_expect_tx(bars + pslot, STAGE);  // the whole box counts, zero fill included
            tma_load_2d(ring + (size_t)pslot * STAGE, &maps.m[item], (int)((pit * Q6K_BYTES) & ~15u), (int)(local * RPT), bars + pslot);
        }
        pslot ^= 1;
        pit += WARPS;
        if (pit >= nblk) {
            pit = warp;
            pt++;
        }
    };
    issue();
    issue();

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    __shared__ TpPushCtx tp_ctx;  // only the first member of a launch may push (tensor-parallel launches are never grouped)
    if (grp.item[0].tp && threadIdx.x == 0) tp_push_ctx_load(&tp_ctx, grp.item[0].tp);
    {
        const uint32_t chunks = nblk * ABLK / 16;
        for (int i = 0; i < grp.count; i++) {
            if (!grp.act_copy[i]) continue;
            const uint8_t *src = (const uint8_t *)grp.item[i].qa;
            uint8_t *dst = acts + grp.act_off[i];
            for (uint32_t c = threadIdx.x; c < chunks; c += THREADS)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s32(dst + 16 * c)), "l"(src + 16 * (size_t)c) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
    }

    const uint32_t colq = (uint32_t)gq < M ? gq : 0;        // activation row of this lane's B fragment
    const uint32_t cp = (uint32_t)(2 * t4) < M ? t4 : 0;    // activation row pair of this lane's C fragment
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

        for (uint32_t it = warp; it < nblk; it += WARPS) {
            if (healthy && !mbar_wait(bars + cslot, cpar)) {
                healthy = false;
                if (lane == 0 && grp.item[0].status) atomicOr(grp.item[0].status, 1);
            }
            if (healthy) {
                const uint8_t *stage = ring + (size_t)cslot * STAGE + ((it * Q6K_BYTES) & 15u);
                const uint8_t *ab = iacts + (size_t)it * ABLK;
                const float2 *dsp = (const float2 *)(ab + 256 * M) + 2 * cp;  // {da[c0], da[c1]} of sub-block s at [8 * (s >> 1) + (s & 1)]
#pragma unroll
                for (int tl = 0; tl < TILES; tl++) {
                    const uint8_t *b0 = stage + (tl * 16 + gq) * BOX, *b1 = b0 + 8 * BOX;  // this lane's two weight rows
                    // int8 sub-scales of both rows: 16 bytes each, as four words
                    uint32_t s0[4], s1[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        s0[i] = lds_u32_align2(b0 + 192 + 4 * i);
                        s1[i] = lds_u32_align2(b1 + 192 + 4 * i);
                    }
                    float blk[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // sum over the block's groups of (sc-weighted dots) * da
#pragma unroll
                    for (int nh = 0; nh < 2; nh++) {
                        // the two high bits of 32 weights x 4 sub-blocks live in one qh byte each: load once per (half, 16-group)
                        uint32_t h0[2], h1[2];
#pragma unroll
                        for (int g = 0; g < 2; g++) {
                            h0[g] = lds_u32_align2(b0 + 128 + 32 * nh + 16 * g + 4 * t4) ^ 0xAAAAAAAAu;  // top bit of every 2-bit field flipped: see header
                            h1[g] = lds_u32_align2(b1 + 128 + 32 * nh + 16 * g + 4 * t4) ^ 0xAAAAAAAAu;
                        }
#pragma unroll
                        for (int tt = 0; tt < 4; tt++) {  // sub-block 4 nh + tt of the super-block = activation group
                            const int s = 4 * nh + tt;
                            int tsum[4] = {0, 0, 0, 0};
#pragma unroll
                            for (int g = 0; g < 2; g++) {  // its two 16-weight groups, each with its own scale
                                const uint32_t l0 = lds_u32_align2(b0 + 64 * nh + 32 * (tt & 1) + 16 * g + 4 * t4);
                                const uint32_t l1 = lds_u32_align2(b1 + 64 * nh + 32 * (tt & 1) + 16 * g + 4 * t4);
                                // 4 * (q - 32) as int8: nibble -> bits 2..5, high bits -> bits 6..7
                                const uint32_t n0 = (tt < 2 ? (l0 << 2) : (l0 >> 2)) & 0x3C3C3C3Cu;
                                const uint32_t n1 = (tt < 2 ? (l1 << 2) : (l1 >> 2)) & 0x3C3C3C3Cu;
                                const uint32_t a0 = ((tt == 3 ? h0[g] : (h0[g] << (6 - 2 * tt))) & 0xC0C0C0C0u) | n0;
                                const uint32_t a1 = ((tt == 3 ? h1[g] : (h1[g] << (6 - 2 * tt))) & 0xC0C0C0C0u) | n1;
                                const uint32_t bq = *(const uint32_t *)(ab + s * (M * 32) + colq * 32 + 16 * g + 4 * t4);
                                int c[4];
                                mma_s8_k16(c, a0, a1, bq);
                                const int is = 8 * nh + 2 * tt + g;  // sub-scale index inside the block
                                const int sc0 = sbyte(s0[is >> 2], is & 3), sc1 = sbyte(s1[is >> 2], is & 3);
                                tsum[0] += sc0 * c[0];
                                tsum[1] += sc0 * c[1];
                                tsum[2] += sc1 * c[2];
                                tsum[3] += sc1 * c[3];
                            }
                            const float2 da = dsp[8 * (s >> 1) + (s & 1)];
                            blk[0] = fmaf((float)tsum[0], da.x, blk[0]);
                            blk[1] = fmaf((float)tsum[1], da.y, blk[1]);
                            blk[2] = fmaf((float)tsum[2], da.x, blk[2]);
                            blk[3] = fmaf((float)tsum[3], da.y, blk[3]);
                        }
                    }
                    // d / 4: the weights went in as 4 * (q - 32)
                    const float d0 = half_bits_to_float(*(const uint16_t *)(b0 + 208)) * 0.25f;
                    const float d1 = half_bits_to_float(*(const uint16_t *)(b1 + 208)) * 0.25f;
                    acc[tl][0] = fmaf(d0, blk[0], acc[tl][0]);
                    acc[tl][1] = fmaf(d0, blk[1], acc[tl][1]);
                    acc[tl][2] = fmaf(d1, blk[2], acc[tl][2]);
                    acc[tl][3] = fmaf(d1, blk[3], acc[tl][3]);
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
}

struct Config {
    int warps, tiles;
};
static const Config CONFIGS[] = {{8, 2}, {8, 1}, {4, 1}};

static size_t fixed_smem(const Config &c) {
    const size_t stage = (size_t)16 * c.tiles * BOX;
    return BAR_BYTES + (size_t)c.warps * STAGES * stage + (size_t)2 * c.warps * 16 * c.tiles * 8 * 4;
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

static int g_force_config = -1;  // tuning: -1 = choose
static double g_balance_margin = 1.08;

static int pick_config(size_t act_bytes) {
    if (g_force_config >= 0 && fixed_smem(CONFIGS[g_force_config]) + act_bytes <= 227 * 1024 - 256) return g_force_config;
    for (int i = 0; i < (int)(sizeof(CONFIGS) / sizeof(CONFIGS[0])); i++)
        if (fixed_smem(CONFIGS[i]) + act_bytes <= 227 * 1024 - 256) return i;
    return -1;
}

// The launch's layout: the first that fits, unless the next one shares the row tiles among the CTAs more evenly by a
// margin that outweighs what its 16-row warps lose (they load every activation fragment once per 16 instead of once
// per 32 rows): 14336 rows are 448 tiles of 32 = rounds of 4 and 3 over 148 CTAs, but 896 of 16 = rounds of 7 and 6.
static int pick_config_for(const GemvGroup &g, int sm_count) {
    const int first = pick_config(g.act_bytes);
    if (first != 0 || g_force_config >= 0 || fixed_smem(CONFIGS[1]) + g.act_bytes > 227 * 1024 - 256) return first;
    auto eff = [&](int tiles) {
        uint64_t tasks = 0;
        for (int i = 0; i < g.count; i++) tasks += (g.item[i].n + 16 * tiles - 1) / (16 * tiles);
        const uint64_t grid = tasks < (uint64_t)sm_count ? tasks : (uint64_t)sm_count;
        return (double)tasks / ((double)grid * ((tasks + grid - 1) / grid));
    };
    return eff(1) > g_balance_margin * eff(2) ? 1 : 0;
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

// A tensor map depends only on (address, n, k, box rows): the last few are remembered.
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
    cuuint64_t dims[2] = {(cuuint64_t)nblk * Q6K_BYTES, a.n};
    cuuint64_t strides[1] = {(cuuint64_t)nblk * Q6K_BYTES};
    cuuint32_t box[2] = {BOX, box_rows};
    cuuint32_t es[2] = {1, 1};
    if (enc(&out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)a.w, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
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

template <int WARPS, int TILES, int NG>
static cudaError_t launch_n(GemvGroupT<NG> &g, int sm_count, bool pdl, cudaStream_t stream) {
    auto kern = qgemv_q6k_mma_kernel<WARPS, TILES, NG>;
    uint32_t tasks = 0;
    WeightMapsT<NG> maps;
    for (int i = 0; i < g.count; i++) {
        tasks += (g.item[i].n + 16 * TILES - 1) / (16 * TILES);
        g.task_end[i] = tasks;
        if (!weight_map(g.item[i], 16 * TILES, maps.m[i])) return cudaErrorNotSupported;
    }
    for (int i = g.count; i < NG; i++) maps.m[i] = maps.m[0];
    const size_t smem = fixed_smem(Config{WARPS, TILES}) + g.act_bytes;
    static DynamicSmemOptIn opted;
    if (cudaError_t e = opted.raise((const void *)kern, smem); e != cudaSuccess) return e;
    const uint32_t per_sm = (uint32_t)((227 * 1024) / (smem + 1024));  // shared memory is what limits residency
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

template <int WARPS, int TILES>
static cudaError_t launch_cfg(GemvGroup &g, int sm_count, bool pdl, cudaStream_t stream) {
    if (g.count > 1) return launch_n<WARPS, TILES, GEMV_GROUP_MAX>(g, sm_count, pdl, stream);
    GemvSingle one;  // a lone launch passes a sixth of the parameter bytes
    one.item[0] = g.item[0];
    one.act_off[0] = g.act_off[0];
    one.act_copy[0] = g.act_copy[0];
    one.count = 1;
    one.act_bytes = g.act_bytes;
    return launch_n<WARPS, TILES, 1>(one, sm_count, pdl, stream);
}

}  // namespace m6

void qgemv_q6k_mma_set_config(int index) { m6::g_force_config = index < 0 || index > 2 ? -1 : index; }

// K a multiple of 2048: a row of the packed matrix must be a multiple of 16 bytes for the tensor map.
bool qgemv_q6k_mma_shape_ok(uint32_t rows, uint32_t k) {
    if (rows < 1 || rows > 8 || k % QK != 0 || k < QK || (k / QK) % 8 != 0 || !m6::encode_fn()) return false;
    return m6::pick_config((size_t)(k / QK) * m6::act_block_bytes(rows)) >= 0;
}

bool qgemv_q6k_mma_group_fits(GemvGroup &g) {
    m6::plan_acts(g);
    return m6::pick_config(g.act_bytes) >= 0;
}

cudaError_t launch_qgemv_q6k_mma(GemvGroup &g, int sm_count, bool pdl, cudaStream_t stream) {
    if (g.count < 1 || g.count > GEMV_GROUP_MAX) return cudaErrorInvalidValue;
    m6::plan_acts(g);
    switch (m6::pick_config_for(g, sm_count)) {
        case 0: return m6::launch_cfg<8, 2>(g, sm_count, pdl, stream);
        case 1: return m6::launch_cfg<8, 1>(g, sm_count, pdl, stream);
        case 2: return m6::launch_cfg<4, 1>(g, sm_count, pdl, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace lb

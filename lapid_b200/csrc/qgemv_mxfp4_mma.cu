// MXFP4 (ggml `block_mxfp4`: 32 elements in 17 bytes -- an e8m0 scale byte, then 16 bytes whose low nibbles are
// elements 0..15 and high nibbles elements 16..31; x = KV[code] * 2^(e - 128), KV the doubled e2m1 values
// 0, 1, 2, 3, 4, 6, 8, 12 and their negatives; crates/lapid-quant/src/mxfp4.rs:14-25) decode GEMV for 1..8 activation
// rows on the warp-level int8 tensor-core instruction. Arithmetic as in qgemv_mxfp4.cu (lapid-cpu's,
// crates/lapid-cpu/src/mxfp4.rs:38-58): the exact integer dot product of KV with the int8 activations per block, one
// f32 step per block. The sibling of qgemv_i4_mma.cu: same CTA structure (a CTA owns 16-row tiles, its warps split K
// in chunks of 512, stages by cp.async, partial 16x8 tiles summed in warp order, the activation tiles of the K-quant
// kernels).
//
// What differs: a stage is 16 rows x 272 bytes (the chunk's 16 blocks as they lie in memory; K a multiple of 512 makes
// every row and every chunk a multiple of 16 bytes), and a block's nibbles start one byte behind a 17-byte boundary:
// a lane fetches its four bytes as two aligned words and a funnel shift (the row pitch of 68 words spreads the eight
// rows of a fragment over all banks). The int8 operand is made without any per-nibble shuffling:
//  * byte j of a block holds element j (low nibble) and j + 16 (high nibble), so the four nibbles of a 16-bit half
//    are the codes of elements j, j + 16, j + 1, j + 17 -- and four nibbles are exactly what `prmt` takes as its
//    selector. With the sign bits masked off, one `prmt` over the table of magnitudes gives the four |KV|, a second one
//    over the table of negated magnitudes the four -|KV|;
//  * `prmt` of a constant 0x80 bytes with the unmasked half as selector gives 0x80 where a code's sign bit is clear
//    (byte copied) and 0xFF where it is set (top bit replicated); a shift and one logic operation turn that into a
//    byte mask, a last one picks |KV| or -|KV| per byte. The code 8 ("-0") comes out as 0 like any other.
//  * Within a block the k order of an integer dot product is free as long as both operands use the same one: register
//    a0 holds elements (4t, 4t+16, 4t+1, 4t+17), a2 (4t+2, 4t+18, 4t+3, 4t+19), and the activation fragment is brought
//    into the same order with two `prmt` over the lane's two words of the activation tile.
#include "common.cuh"
#include "kernels.h"
#include "tp_ll.cuh"

namespace lb {
namespace mxm {

constexpr int KC = 512;                      // weights per row and stage
constexpr int ROWB = KC / GROUP * MXFP4_BYTES;  // 272 bytes per row and stage
constexpr int STAGE = 16 * ROWB;             // 4352
constexpr int STAGES = 2;
constexpr float MAGIC = 12582912.0f;

__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 16 weight rows x 32 k x 8 activation rows, signed bytes; the accumulators start at the bit
// pattern of 1.5 * 2^23, so the result reinterpreted as f32 is 12582912 + dot (|dot| < 2^22)
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0x4B400000));
}
__host__ __device__ constexpr uint32_t act_block_bytes(uint32_t rows) { return 256 * rows + 512; }  // per 256 k, as the K-quant kernels' tiles

template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 8 ? 2 : 4) qgemv_mxfp4_mma_kernel(GemvArgs p) {
    constexpr int THREADS = WARPS * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gq = lane >> 2, t4 = lane & 3;
    const uint32_t M = p.rows, k = p.k;
    const uint32_t iters = k / KC;
    const uint32_t rowb = k / GROUP * MXFP4_BYTES;  // bytes of a whole weight row
    const uint32_t ABLK = act_block_bytes(M);
    const uint32_t tasks = (p.n + 15) / 16;
    const uint32_t t_lo = (uint32_t)(((uint64_t)tasks * blockIdx.x) / gridDim.x);
    const uint32_t t_hi = (uint32_t)(((uint64_t)tasks * (blockIdx.x + 1)) / gridDim.x);

    uint8_t *ring = smem + (size_t)warp * (STAGES * STAGE);
    float *red = (float *)(smem + (size_t)WARPS * STAGES * STAGE);  // [2][WARPS][128]
    uint8_t *acts = (uint8_t *)(red + 2 * WARPS * 128);

    // producer cursor: (tile, chunk, ring slot). One stage = 16 rows x 17 sixteen-byte copies, 8.5 per lane.
    uint32_t pt = t_lo, pit = warp, pslot = 0;
    auto issue = [&]() {
        if (pt < t_hi && (uint32_t)warp < iters) {
            uint8_t *dst = ring + (size_t)pslot * STAGE;
            const uint32_t row0 = pt * 16;
#pragma unroll
            for (int i = 0; i < 9; i++) {
                const uint32_t idx = i * 32 + lane;
                if (idx < 16 * 17) {
                    const uint32_t r = idx / 17, c = idx % 17;
                    const uint32_t row = min(row0 + r, p.n - 1);  // rows past the end repeat the last one; their outputs are dropped
                    const uint8_t *src = p.w + (size_t)row * rowb + (size_t)pit * ROWB + 16 * c;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s32(dst + r * ROWB + 16 * c)), "l"(src) : "memory");
                }
            }
            pslot ^= 1;
            pit += WARPS;
            if (pit >= iters) {
                pit = warp;
                pt++;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");  // an empty group keeps the count in step
    };
    issue();
    issue();

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    __shared__ TpPushCtx tp_ctx;
    if (p.tp && threadIdx.x == 0) tp_push_ctx_load(&tp_ctx, p.tp);
    {   // the activation tiles, once per CTA (their own cp.async group, waited for with the first stage)
        const uint32_t chunks = (k / QK) * ABLK / 16;
        const uint8_t *src = (const uint8_t *)p.qa;
        for (uint32_t c = threadIdx.x; c < chunks; c += THREADS)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s32(acts + 16 * c)), "l"(src + 16 * (size_t)c) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
    }

    const uint32_t colq = (uint32_t)gq < M ? gq : 0;      // activation row of this lane's B fragment
    const uint32_t cp = (uint32_t)(2 * t4) < M ? t4 : 0;  // activation row pair of this lane's C fragment
    uint32_t cslot = 0, par = 0;
    for (uint32_t t = t_lo; t < t_hi; t++, par ^= 1) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (uint32_t it = warp; it < iters; it += WARPS) {
            asm volatile("cp.async.wait_group 1;" ::: "memory");  // all but the newest group: this stage has landed
            __syncwarp();
            const uint8_t *stage = ring + (size_t)cslot * STAGE;
            const uint8_t *row_lo = stage + gq * ROWB, *row_hi = stage + (gq + 8) * ROWB;
#pragma unroll
            for (int blk = 0; blk < 2; blk++) {  // the chunk's two 256-wide activation tiles
                const uint8_t *ab = acts + (size_t)(2 * it + blk) * ABLK;
                const float2 *dsp = (const float2 *)(ab + 256 * M) + 2 * cp;  // {da[c0], da[c1]} of group s at [8 * (s >> 1) + (s & 1)]
#pragma unroll
                for (int s = 0; s < 8; s++) {
                    const uint32_t off = (uint32_t)(8 * blk + s) * MXFP4_BYTES;  // this block inside the row's 272 bytes
                    // bytes 4 t4 .. 4 t4 + 3 of the block's 16 nibble bytes: two aligned words around them
                    const uint32_t at = off + 1 + 4 * t4, sh = (at & 3u) * 8u;
                    const uint32_t *pl = (const uint32_t *)(row_lo + (at & ~3u)), *ph = (const uint32_t *)(row_hi + (at & ~3u));
                    const uint32_t wl = __funnelshift_r(pl[0], pl[1], sh), wh = __funnelshift_r(ph[0], ph[1], sh);
                    const uint32_t a0 = mxfp4_kv4(wl), a2 = mxfp4_kv4(wl >> 16), a1 = mxfp4_kv4(wh), a3 = mxfp4_kv4(wh >> 16);
                    // the activations of elements 4 t4 .. and 16 + 4 t4 .., brought into the same order
                    const uint8_t *bp = ab + s * (M * 32) + colq * 32 + 4 * t4;
                    const uint32_t bl = *(const uint32_t *)bp, bh = *(const uint32_t *)(bp + 16);
                    int c[4];
                    mma_s8(c, a0, a1, a2, a3, prmt(bl, bh, 0x5140u), prmt(bl, bh, 0x7362u));
                    const float2 da = dsp[8 * (s >> 1) + (s & 1)];
                    const float w0 = e8m0_half(row_lo[off]), w1 = e8m0_half(row_hi[off]);
                    acc[0] = fmaf((__int_as_float(c[0]) - MAGIC) * da.x, w0, acc[0]);
                    acc[1] = fmaf((__int_as_float(c[1]) - MAGIC) * da.y, w0, acc[1]);
                    acc[2] = fmaf((__int_as_float(c[2]) - MAGIC) * da.x, w1, acc[2]);
                    acc[3] = fmaf((__int_as_float(c[3]) - MAGIC) * da.y, w1, acc[3]);
                }
            }
            __syncwarp();  // every lane is done reading the slot before it is refilled
            issue();
            cslot ^= 1;
        }
        if ((uint32_t)warp >= iters) issue();  // keeps idle warps' (empty) group count in step; they never wait

        // ---- sum the warps' partial tiles (warp order) and store: one output per thread
        float *mine = red + ((size_t)par * WARPS + warp) * 128;
#pragma unroll
        for (int i = 0; i < 4; i++) mine[i * 32 + lane] = acc[i];
        __syncthreads();  // the buffer of the other parity is free again once every warp got here
        for (uint32_t e = threadIdx.x; e < 128; e += THREADS) {
            const float *src = red + (size_t)par * WARPS * 128 + e;
            float v = src[0];
#pragma unroll
            for (int w = 1; w < WARPS; w++) v += src[(size_t)w * 128];
            const uint32_t el = e & 31, i = e >> 5;
            const uint32_t row = t * 16 + (el >> 2) + ((i & 2) ? 8 : 0);
            const uint32_t r = 2 * (el & 3) + (i & 1);
            if (row < p.n && r < M) {
                const uint32_t bt = r / p.m, ri = r % p.m;
                if (p.extra && !p.epi.n) v += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)ri * p.ex_s1 + (int64_t)row * p.ex_s2];
                if (p.tp) tp_push_value(&tp_ctx, (uint64_t)r * p.n + row, v);  // row-parallel partial: to every rank
                else p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)ri * p.out_rs + row] = v;
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

static size_t smem_bytes(int warps, uint32_t rows, uint32_t k) {
    return (size_t)warps * (STAGES * STAGE + 2 * 128 * 4) + (size_t)(k / QK) * act_block_bytes(rows) + 16;
}

template <int WARPS> static cudaError_t launch_w(const GemvArgs &a, int sm_count, bool pdl, cudaStream_t stream) {
    auto kern = qgemv_mxfp4_mma_kernel<WARPS>;
    const size_t smem = smem_bytes(WARPS, a.rows, a.k);
    static DynamicSmemOptIn opted;
    if (cudaError_t e = opted.raise((const void *)kern, smem); e != cudaSuccess) return e;
    const uint32_t tasks = (a.n + 15) / 16;
    uint32_t fit = (uint32_t)((227 * 1024) / (smem + 1024));
    if (fit < 1) fit = 1;
    // CTAs per SM: the count whose equal shares of the 16-row tiles are the most even; more CTAs on a tie
    uint32_t grid = 1;
    double best = 0.0;
    for (uint32_t c = 1; c <= fit && c <= 4; c++) {
        uint32_t g = (uint32_t)sm_count * c;
        if (g > tasks) g = tasks;
        const double eff = (double)tasks / ((double)g * ((tasks + g - 1) / g));
        if (eff >= best) best = eff, grid = g;
    }
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
    return cudaLaunchKernelEx(&cfg, kern, a);
}

}  // namespace mxm

// K a multiple of 512: whole stages, and every row and chunk of the packed matrix a multiple of 16 bytes.
bool qgemv_mxfp4_mma_shape_ok(uint32_t rows, uint32_t k) {
    if (rows < 1 || rows > 8 || k < mxm::KC || k % mxm::KC != 0) return false;
    return mxm::smem_bytes(4, rows, k) <= 227 * 1024 - 256;
}

cudaError_t launch_qgemv_mxfp4_mma(const GemvArgs &a, int sm_count, bool pdl, cudaStream_t stream) {
    if (!qgemv_mxfp4_mma_shape_ok(a.rows, a.k) || ((uintptr_t)a.w & 15) != 0) return cudaErrorInvalidValue;
    if (mxm::smem_bytes(8, a.rows, a.k) <= 227 * 1024 - 256) return mxm::launch_w<8>(a, sm_count, pdl, stream);
    return mxm::launch_w<4>(a, sm_count, pdl, stream);
}

}  // namespace lb

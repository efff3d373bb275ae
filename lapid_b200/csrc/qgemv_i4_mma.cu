// Int4 (GGUF Q4_0 in lapid's plane layout: per 32-element group 16 bytes, byte j = element j in the low and element
// j + 16 in the high nibble, x = (q - 8) * d with an f16 scale per group; crates/lapid-quant/src/lib.rs:5-17) decode GEMV
// for 2..8 activation rows on the warp-level int8 tensor-core instruction. The sibling of qgemv_i8_mma.cu (same CTA
// structure: warps split K in chunks of 512, stages by cp.async, partial 16x8 tiles summed in warp order, the
// activation tiles of the K-quant kernels); arithmetic as in qgemv_i4.cu: the exact integer dot product of (q - 8)
// with the int8 activations per group, one f32 step per group (crates/lapid-cpu/src/matmul/qkernels.rs:60-84 through
// crates/lapid-cpu/src/qmat.rs:97-112).
//
// What differs from Int8: a stage is 16 rows x 256 bytes of nibbles (plus the 16 x 16 f16 scales), and the MMA's A
// operand is made from it with two logic operations per register: (q ^ 8) is the 4-bit two's complement of q - 8, so
// that nibble in the HIGH half of a byte is the int8 value 16 (q - 8) -- `(w << 4 & 0xF0F0F0F0) ^ 0x80808080` for the low
// nibbles, `(w & 0xF0F0F0F0) ^ 0x80808080` for the high ones -- and the exact factor 1/16 goes into the group's scale.
// Within a group the k order is free as long as both operands agree: lane t takes elements 8t..8t+7, which are the low
// nibbles of bytes 8t..8t+7 for t = 0, 1 and the high nibbles of bytes 8(t-2).. for t = 2, 3 (one 64-bit load either
// way). 16-byte chunk c of row r sits at chunk position c ^ (r & 7), which makes those loads bank-conflict free.
#include "common.cuh"
#include "kernels.h"
#include "tp_ll.cuh"

namespace lb {
namespace i4m {

constexpr int KC = 512;                        // weights per row and stage
constexpr int ROWB = KC / 2;                   // bytes of nibbles per row and stage
constexpr int Q_BYTES = 16 * ROWB;             // 4096
constexpr int STAGE = Q_BYTES + 16 * (KC / 16);  // + 16 rows x 32 bytes of f16 scales = 4608
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
__global__ void __launch_bounds__(WARPS * 32, 1) qgemv_i4_mma_kernel(GemvArgs p) {
    constexpr int THREADS = WARPS * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gq = lane >> 2, t4 = lane & 3;
    const uint32_t M = p.rows, k = p.k, kg = k / GROUP;
    const uint32_t iters = k / KC;
    const uint32_t ABLK = act_block_bytes(M);
    const uint32_t tasks = (p.n + 15) / 16;
    const uint32_t t_lo = (uint32_t)(((uint64_t)tasks * blockIdx.x) / gridDim.x);
    const uint32_t t_hi = (uint32_t)(((uint64_t)tasks * (blockIdx.x + 1)) / gridDim.x);
    const uint8_t *wq = p.w;
    const uint8_t *ws = p.w + p.scales_offset;

    uint8_t *ring = smem + (size_t)warp * (STAGES * STAGE);
    float *red = (float *)(smem + (size_t)WARPS * STAGES * STAGE);  // [2][WARPS][128]
    uint8_t *acts = (uint8_t *)(red + 2 * WARPS * 128);

    // producer cursor: (tile, chunk, ring slot). One stage = 256 + 32 sixteen-byte copies, 9 per lane.
    uint32_t pt = t_lo, pit = warp, pslot = 0;
    auto issue = [&]() {
        if (pt < t_hi && (uint32_t)warp < iters) {
            uint8_t *dst = ring + (size_t)pslot * STAGE;
            const uint32_t row0 = pt * 16;
#pragma unroll
            for (int i = 0; i < 8; i++) {  // nibbles: lane -> 16-byte chunk (lane & 15) of row 2 i + (lane >> 4)
                const uint32_t r = 2 * i + (lane >> 4), c = lane & 15;
                const uint32_t row = min(row0 + r, p.n - 1);  // rows past the end repeat the last one; their outputs are dropped
                const uint8_t *src = wq + (size_t)row * (k / 2) + (size_t)pit * ROWB + 16 * c;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s32(dst + r * ROWB + 16 * (c ^ (r & 7)))), "l"(src) : "memory");
            }
            {   // scales: lane -> half (lane & 1) of row lane / 2
                const uint32_t row = min(row0 + (lane >> 1), p.n - 1);
                const uint8_t *src = ws + ((size_t)row * kg + (size_t)pit * (KC / GROUP)) * 2 + 16 * (lane & 1);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s32(dst + Q_BYTES + 16 * lane)), "l"(src) : "memory");
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
#pragma unroll
            for (int blk = 0; blk < 2; blk++) {  // the chunk's two 256-wide activation tiles
                const uint8_t *ab = acts + (size_t)(2 * it + blk) * ABLK;
                const float2 *dsp = (const float2 *)(ab + 256 * M) + 2 * cp;  // {da[c0], da[c1]} of group s at [8 * (s >> 1) + (s & 1)]
                // the f16 scales of this lane's two weight rows for the tile's eight groups
                const uint4 sw0 = *(const uint4 *)(stage + Q_BYTES + gq * 32 + 16 * blk);
                const uint4 sw1 = *(const uint4 *)(stage + Q_BYTES + (gq + 8) * 32 + 16 * blk);
                const uint32_t s0[4] = {sw0.x, sw0.y, sw0.z, sw0.w}, s1[4] = {sw1.x, sw1.y, sw1.z, sw1.w};
#pragma unroll
                for (int s = 0; s < 8; s++) {
                    const int c16 = 8 * blk + s;  // the group's 16 bytes are one chunk of the row
                    const uint2 w_lo = *(const uint2 *)(stage + gq * ROWB + 16 * (c16 ^ (gq & 7)) + 8 * (t4 & 1));
                    const uint2 w_hi = *(const uint2 *)(stage + (gq + 8) * ROWB + 16 * (c16 ^ (gq & 7)) + 8 * (t4 & 1));
                    const uint2 b = *(const uint2 *)(ab + s * (M * 32) + colq * 32 + 8 * t4);
                    // 16 (q - 8) as int8: low nibbles (elements 0..15 of the group) for t4 < 2, high nibbles above
                    const int sh = t4 < 2 ? 4 : 0;
                    const uint32_t a0 = ((w_lo.x << sh) & 0xF0F0F0F0u) ^ 0x80808080u, a2 = ((w_lo.y << sh) & 0xF0F0F0F0u) ^ 0x80808080u;
                    const uint32_t a1 = ((w_hi.x << sh) & 0xF0F0F0F0u) ^ 0x80808080u, a3 = ((w_hi.y << sh) & 0xF0F0F0F0u) ^ 0x80808080u;
                    int c[4];
                    mma_s8(c, a0, a1, a2, a3, b.x, b.y);
                    const float2 da = dsp[8 * (s >> 1) + (s & 1)];
                    const float w0 = half_bits_to_float((s0[s >> 1] >> (16 * (s & 1))) & 0xffff) * 0.0625f;  // (the dot is 16 times too large)
                    const float w1 = half_bits_to_float((s1[s >> 1] >> (16 * (s & 1))) & 0xffff) * 0.0625f;
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
    return (size_t)warps * (STAGES * STAGE + 2 * 128 * 4) + (size_t)(k / QK) * act_block_bytes(rows);
}

template <int WARPS> static cudaError_t launch_w(const GemvArgs &a, int sm_count, bool pdl, cudaStream_t stream) {
    auto kern = qgemv_i4_mma_kernel<WARPS>;
    const size_t smem = smem_bytes(WARPS, a.rows, a.k);
    static DynamicSmemOptIn opted;
    if (cudaError_t e = opted.raise((const void *)kern, smem); e != cudaSuccess) return e;
    const uint32_t tasks = (a.n + 15) / 16;
    uint32_t fit = (uint32_t)((227 * 1024) / (smem + 1024));
    if (fit < 1) fit = 1;
    // CTAs per SM: the count whose equal shares of the 16-row tiles are the most even (896 tiles over 296 CTAs are
    // rounds of 4 and 3: a quarter of the time half the GPU idles; over 148 they are 7 and 6); more CTAs on a tie
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

}  // namespace i4m

// K a multiple of 512 (whole stages; also makes every 16-byte copy of nibbles and scales aligned).
bool qgemv_i4_mma_shape_ok(uint32_t rows, uint32_t k) {
    if (rows < 1 || rows > 8 || k < i4m::KC || k % i4m::KC != 0) return false;
    return i4m::smem_bytes(4, rows, k) <= 227 * 1024 - 256;
}

cudaError_t launch_qgemv_i4_mma(const GemvArgs &a, int sm_count, bool pdl, cudaStream_t stream) {
    if (!qgemv_i4_mma_shape_ok(a.rows, a.k) || ((uintptr_t)a.w & 15) != 0 || (a.scales_offset & 15) != 0) return cudaErrorInvalidValue;
    if (i4m::smem_bytes(8, a.rows, a.k) <= 227 * 1024 - 256) return i4m::launch_w<8>(a, sm_count, pdl, stream);
    return i4m::launch_w<4>(a, sm_count, pdl, stream);
}

}  // namespace lb

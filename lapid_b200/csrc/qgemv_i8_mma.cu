// Int8 (GGUF Q8_0 in lapid's plane layout) decode GEMV for 2..8 activation rows on the warp-level
// int8 tensor-core instruction. Arithmetic as in qgemv_i8.cu: exact integer dot products per
// 32-element group, one f32 step per group, f32(dot) * da * db (crates/lapid-cpu/src/matmul/
// qkernels.rs:60-84; the order of the two scale multiplications and of the f32 sums differs).
//
// The weights are plain signed bytes, so they are the MMA's A operand as they lie in memory: one
// `mma.sync.m16n8k32.s8.s8` covers 16 weight rows x one 32-element group x 8 activation rows, and
// nothing has to be unpacked. Per CTA the warps split K in chunks of 512 (warp w takes chunks w,
// w + WARPS, ... of the CTA's 16-row tile) and their partial 16x8 tiles are summed in shared memory in
// warp order. A warp's stage is 16 rows x 512 quants plus their 16 x 16 f16 scales, brought in by
// `cp.async` (16 bytes per lane and instruction) into a layout of the kernel's choosing: 16-byte
// chunk c of row r sits at chunk position c ^ 2 (r & 3), which makes the fragment loads (64 bits per
// lane: within a group the k order is free, lane t takes quants 8t..8t+7 of both operands)
// bank-conflict free. Stages of the next chunks are in flight while one is consumed (two per warp,
// cp.async groups), and the first ones are issued before the programmatic-dependent-launch wait.
// Activations: the same shared-memory tiles as the K-quant tensor-core kernels.
#include "common.cuh"
#include "kernels.h"
#include "tp_ll.cuh"

namespace lb {
namespace i8m {

constexpr int KC = 512;                        // quants per row and stage
constexpr int Q_BYTES = 16 * KC;               // 8192
constexpr int STAGE = Q_BYTES + 16 * (KC / 16);  // + 16 rows x 32 bytes of f16 scales = 8704
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
__global__ void __launch_bounds__(WARPS * 32, 1) qgemv_i8_mma_kernel(GemvArgs p) {
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

    // producer cursor: (tile, chunk, ring slot). One stage = 512 + 32 sixteen-byte copies, 17 per lane.
    uint32_t pt = t_lo, pit = warp, pslot = 0;
    auto issue = [&]() {
        if (pt < t_hi && (uint32_t)warp < iters) {
            uint8_t *dst = ring + (size_t)pslot * STAGE;
            const uint32_t row0 = pt * 16;
#pragma unroll
            for (int i = 0; i < 16; i++) {  // quants: lane -> 16-byte chunk `lane` of row i
                const uint32_t row = min(row0 + i, p.n - 1);  // rows past the end repeat the last one; their outputs are dropped
                const uint8_t *src = wq + (size_t)row * k + (size_t)pit * KC + 16 * lane;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s32(dst + i * KC + 16 * (lane ^ (2 * (i & 3))))), "l"(src) : "memory");
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
                    const int c16 = 2 * (8 * blk + s) + (t4 >> 1);  // 16-byte chunk of the row that holds quants 8 t4 .. 8 t4 + 7 of the group
                    const uint2 a_lo = *(const uint2 *)(stage + gq * KC + 16 * (c16 ^ (2 * (gq & 3))) + 8 * (t4 & 1));
                    const uint2 a_hi = *(const uint2 *)(stage + (gq + 8) * KC + 16 * (c16 ^ (2 * (gq & 3))) + 8 * (t4 & 1));
                    const uint2 b = *(const uint2 *)(ab + s * (M * 32) + colq * 32 + 8 * t4);
                    int c[4];
                    mma_s8(c, a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
                    const float2 da = dsp[8 * (s >> 1) + (s & 1)];
                    const float w0 = half_bits_to_float((s0[s >> 1] >> (16 * (s & 1))) & 0xffff);
                    const float w1 = half_bits_to_float((s1[s >> 1] >> (16 * (s & 1))) & 0xffff);
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
    auto kern = qgemv_i8_mma_kernel<WARPS>;
    const size_t smem = smem_bytes(WARPS, a.rows, a.k);
    static DynamicSmemOptIn opted;
    if (cudaError_t e = opted.raise((const void *)kern, smem); e != cudaSuccess) return e;
    const uint32_t tasks = (a.n + 15) / 16;
    uint32_t per_sm = (uint32_t)((227 * 1024) / (smem + 1024));
    if (per_sm < 1) per_sm = 1;
    uint32_t grid = (uint32_t)sm_count * per_sm;
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
    return cudaLaunchKernelEx(&cfg, kern, a);
}

}  // namespace i8m

// K a multiple of 512 (whole stages; also makes every 16-byte copy of quants and scales aligned).
bool qgemv_i8_mma_shape_ok(uint32_t rows, uint32_t k) {
    if (rows < 1 || rows > 8 || k < i8m::KC || k % i8m::KC != 0) return false;
    return i8m::smem_bytes(4, rows, k) <= 227 * 1024 - 256;
}

cudaError_t launch_qgemv_i8_mma(const GemvArgs &a, int sm_count, bool pdl, cudaStream_t stream) {
    if (!qgemv_i8_mma_shape_ok(a.rows, a.k) || ((uintptr_t)a.w & 15) != 0 || (a.scales_offset & 15) != 0) return cudaErrorInvalidValue;
    if (i8m::smem_bytes(8, a.rows, a.k) <= 227 * 1024 - 256) return i8m::launch_w<8>(a, sm_count, pdl, stream);
    return i8m::launch_w<4>(a, sm_count, pdl, stream);
}

}  // namespace lb

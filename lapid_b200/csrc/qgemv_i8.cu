// Int8 (GGUF Q8_0 in lapid's plane layout) decode GEMV, fast path for 1..8 activation rows.
// Arithmetic: acc += f32(sum_32 qa*qb) * (da*db) per 32-group (crates/lapid-cpu/src/matmul/
// qkernels.rs:60-84); here a lane sums 16 of the 32 products, so a group's term is formed as
// f32(dot16)*(da*db) + f32(dot16')*(da*db) -- the integer parts are exact, only f32 rounding of the
// running sum differs (the reference's own AVX2 tile splits a group over eight lanes the same way).
//
// Same machine layout as the K-quant fast path (qgemv_q4k.cu): per-warp rings of shared-memory
// stages filled by `cp.async.bulk`, filled before the programmatic-dependent-launch wait; here a
// stage is up to 4096 quants of one weight row plus their 128 f16 scales (two bulk copies on one
// mbarrier). Quants are plain bytes, so the lane mapping is the simplest one: per step the warp
// reads 512 consecutive quants with one conflict-free 128-bit shared load per lane, the same 16
// activation quants per row, and issues four `dp4a`. The quantized activations (planes written by
// the pre-pass) are copied to shared memory once per CTA.
#include "common.cuh"
#include "kernels.h"

namespace lb {
namespace i8 {

constexpr int CHUNK = 4096;                 // quants per stage
constexpr int STAGE = CHUNK + CHUNK / 16;   // + 2 bytes of scale per 32 quants = 4352
constexpr int BAR_BYTES = 256;
template <int M> struct Shape { static constexpr int WARPS = M <= 2 ? 4 : 8, MIN_CTAS = M <= 2 ? 5 : 2; };

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

// EARLY (one row; GemvArgs::early): the activations are older than the kernel in front of this one, so the
// kernel reads and computes without waiting for it, parks its results in shared memory and stores them
// after the dependency wait; launched as one CTA per SM so that consecutive launches share the SMs
// (see qgemv_q4k.cu).
constexpr int PEND_ROWS = 32;  // parked results per warp
// I4: the same kernel over Int4 nibble planes (GGUF Q4_0 in lapid's plane layout: 16 bytes per 32-element group, byte j =
// element j in the low and element j + 16 in the high nibble, x = (q - 8) * d; crates/lapid-quant/src/lib.rs:5-17,
// crates/lapid-cpu/src/qmat.rs:97-112). A stage holds the nibbles of the same 4096 weights (2048 bytes) and their
// scales; a lane takes one whole group per step (16 bytes), turns each nibble into the int8 value 16 (q - 8) with two
// logic operations per word (the nibble moved into the high half of its byte, its top bit flipped) and multiplies
// with eight `dp4a`; the exact factor 1/16 goes into the scale.
template <int M, bool EARLY = false, bool I4 = false>
__global__ void __launch_bounds__(Shape<M>::WARPS * 32, Shape<M>::MIN_CTAS) qgemv_i8_fast_kernel(GemvArgs p) {
    static_assert(!EARLY || M == 1, "early mode is built for one row");
    constexpr int WARPS = Shape<M>::WARPS, THREADS = WARPS * 32, STAGES = 2;
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t n = p.n, k = p.k, kg = k / GROUP;
    const uint32_t chunks = (k + CHUNK - 1) / CHUNK;
    const uint32_t t_lo = (uint32_t)(((uint64_t)n * blockIdx.x) / gridDim.x);
    const uint32_t t_hi = (uint32_t)(((uint64_t)n * (blockIdx.x + 1)) / gridDim.x);

    uint64_t *bars = (uint64_t *)smem + warp * STAGES;
    uint8_t *ring = smem + BAR_BYTES + (size_t)warp * (STAGES * STAGE);
    uint8_t *act_q = smem + BAR_BYTES + (size_t)WARPS * STAGES * STAGE;  // int8 [rows][k]
    float *act_d = (float *)(act_q + (size_t)p.rows * k);               // f32 [rows][k/32]

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) mbar_init(bars + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    uint32_t pt = t_lo + warp, pc = 0, pslot = 0;  // producer cursor: weight row, chunk, slot
    auto issue = [&]() {
        if (pt >= t_hi) return;
        if (lane == 0) {
            const uint32_t e0 = pc * CHUNK, len = min((uint32_t)CHUNK, k - e0);
            uint8_t *dst = ring + (size_t)pslot * STAGE;
            const uint32_t qbytes = I4 ? len / 2 : len;
            mbar_expect_tx(bars + pslot, qbytes + len / 16);
            bulk_g2s(dst, p.w + (I4 ? ((uint64_t)pt * k + e0) / 2 : (uint64_t)pt * k + e0), qbytes, bars + pslot);
            bulk_g2s(dst + CHUNK, p.w + p.scales_offset + ((uint64_t)pt * kg + e0 / GROUP) * 2, len / 16, bars + pslot);
        }
        pslot ^= 1;
        if (++pc == chunks) {
            pc = 0;
            pt += WARPS;
        }
    };
    issue();
    issue();

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if constexpr (!EARLY) asm volatile("griddepcontrol.wait;" ::: "memory");
    bool waited = !EARLY;
    float *pend = act_d + (size_t)p.rows * kg + warp * PEND_ROWS;  // EARLY: behind the activation scales
    uint32_t npend = 0;
    const uint32_t pend_first = t_lo + warp;
    auto flush_pending = [&]() {
        if (lane == 0)
            for (uint32_t q = 0; q < npend; q++) {
                const uint32_t row = pend_first + q * WARPS;
                float v = pend[q];
                if (p.extra && !p.epi.n) v += p.extra[p.ex_off + (int64_t)row * p.ex_s2];
                p.out[p.out_off + row] = v;
            }
        npend = 0;
    };
    {
        const uint32_t qchunks = p.rows * k / 16, dchunks = p.rows * kg / 4;
        for (uint32_t c = threadIdx.x; c < qchunks; c += THREADS)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s32(act_q + 16 * c)), "l"((const uint8_t *)p.qa + 16 * (size_t)c) : "memory");
        for (uint32_t c = threadIdx.x; c < dchunks; c += THREADS)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s32((uint8_t *)act_d + 16 * c)), "l"((const uint8_t *)p.da + 16 * (size_t)c) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
    }

    bool healthy = true;
    uint32_t cslot = 0, cpar = 0;
    for (uint32_t row = t_lo + warp; row < t_hi; row += WARPS) {
        float acc[M];
#pragma unroll
        for (int r = 0; r < M; r++) acc[r] = 0.0f;
        for (uint32_t c = 0; c < chunks; c++) {
            if (healthy && !mbar_wait(bars + cslot, cpar)) {
                healthy = false;
                if (lane == 0 && p.status) atomicOr(p.status, 1);
            }
            const uint32_t e0 = c * CHUNK, len = min((uint32_t)CHUNK, k - e0);
            const uint8_t *st = ring + (size_t)cslot * STAGE;
            if (healthy && I4) {
                for (uint32_t u = 0; u < len; u += 1024) {  // a group per lane: 1024 weights per warp step
                    if (u + 32 * lane >= len) continue;      // (K is a multiple of 512: the last step may be half empty)
                    const uint4 wq = *(const uint4 *)(st + (u >> 1) + 16 * lane);
                    const float db = half_bits_to_float(*(const uint16_t *)(st + CHUNK + 2 * ((u >> 5) + lane))) * 0.0625f;
                    const uint32_t kk = e0 + u + 32 * lane;  // first of this lane's 32 k
                    const uint32_t w4[4] = {wq.x, wq.y, wq.z, wq.w};
                    uint32_t lo[4], hi[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        lo[i] = ((w4[i] << 4) & 0xF0F0F0F0u) ^ 0x80808080u;  // 16 (q - 8), elements 4i .. 4i + 3
                        hi[i] = (w4[i] & 0xF0F0F0F0u) ^ 0x80808080u;         // elements 16 + 4i ..
                    }
#pragma unroll
                    for (int r = 0; r < M; r++) {
                        const uint4 a0 = *(const uint4 *)(act_q + (size_t)r * k + kk), a1 = *(const uint4 *)(act_q + (size_t)r * k + kk + 16);
                        const float da = act_d[(size_t)r * kg + (kk >> 5)];
                        int dsum = __dp4a((int)lo[0], (int)a0.x, 0);
                        dsum = __dp4a((int)lo[1], (int)a0.y, dsum);
                        dsum = __dp4a((int)lo[2], (int)a0.z, dsum);
                        dsum = __dp4a((int)lo[3], (int)a0.w, dsum);
                        dsum = __dp4a((int)hi[0], (int)a1.x, dsum);
                        dsum = __dp4a((int)hi[1], (int)a1.y, dsum);
                        dsum = __dp4a((int)hi[2], (int)a1.z, dsum);
                        dsum = __dp4a((int)hi[3], (int)a1.w, dsum);
                        acc[r] = fmaf((float)dsum, da * db, acc[r]);
                    }
                }
            }
            if (healthy && !I4) {
                for (uint32_t u = 0; u < len; u += 512) {
                    const uint4 wq = *(const uint4 *)(st + u + 16 * lane);
                    const float db = half_bits_to_float(*(const uint16_t *)(st + CHUNK + 2 * ((u >> 5) + (lane >> 1))));
                    const uint32_t kk = e0 + u + 16 * lane;  // first of this lane's 16 k
#pragma unroll
                    for (int r = 0; r < M; r++) {
                        const uint4 aq = *(const uint4 *)(act_q + (size_t)r * k + kk);
                        const float da = act_d[(size_t)r * kg + (kk >> 5)];
                        int dsum = __dp4a((int)wq.x, (int)aq.x, 0);
                        dsum = __dp4a((int)wq.y, (int)aq.y, dsum);
                        dsum = __dp4a((int)wq.z, (int)aq.z, dsum);
                        dsum = __dp4a((int)wq.w, (int)aq.w, dsum);
                        acc[r] = fmaf((float)dsum, da * db, acc[r]);
                    }
                }
            }
            __syncwarp();
            issue();
            cslot ^= 1;
            if (cslot == 0) cpar ^= 1;
        }
        if (EARLY && !waited) {  // park the result: nothing is written before the kernel in front has completed
            float v = acc[0];
#pragma unroll
            for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) pend[npend] = v;
            if (++npend == PEND_ROWS) {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                waited = true;
                flush_pending();
            }
            continue;
        }
#pragma unroll
        for (int r = 0; r < M; r++) {
            float v = acc[r];
#pragma unroll
            for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) {
                const uint32_t bt = r / p.m, i = r % p.m;
                if (p.extra && !p.epi.n) v += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)i * p.ex_s1 + (int64_t)row * p.ex_s2];
                p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)i * p.out_rs + row] = v;
            }
        }
    }
    if (!waited) {  // (a CTA without a row must not let the grid end before the kernel in front either)
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if constexpr (EARLY) flush_pending();
    }
}

template <int M, bool EARLY = false, bool I4 = false> static cudaError_t launch_m(const GemvArgs &a, int sm_count, bool pdl, cudaStream_t stream) {
    if constexpr (M == 1 && !EARLY) {
        if (pdl && a.early && !a.tp) return launch_m<M, true, I4>(a, sm_count, pdl, stream);
    }
    auto kern = qgemv_i8_fast_kernel<M, EARLY, I4>;
    constexpr int WARPS = Shape<M>::WARPS;
    const size_t smem = BAR_BYTES + (size_t)WARPS * 2 * STAGE + (size_t)a.rows * a.k + (size_t)a.rows * (a.k / GROUP) * 4 +
                        (EARLY ? (size_t)WARPS * PEND_ROWS * 4 : 0);
    static DynamicSmemOptIn opted;
    if (cudaError_t e = opted.raise((const void *)kern, smem); e != cudaSuccess) return e;
    static OccupancyCache occupancy;
    int ctas_per_sm = 1;
    if (cudaError_t e = occupancy.get(kern, WARPS * 32, smem, &ctas_per_sm); e != cudaSuccess) return e;
    int per_sm = ctas_per_sm >= 4 ? ctas_per_sm - 1 : ctas_per_sm;  // one slot for the next kernel (see qgemv_q4k.cu)
    if (EARLY) per_sm = 1;                                          // the other slots belong to the launches around this one
    uint32_t grid = (uint32_t)sm_count * (uint32_t)per_sm;
    const uint32_t useful = (a.n + WARPS - 1) / WARPS;
    if (grid > useful) grid = useful;
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

}  // namespace i8

// K must be a multiple of 512 (one warp step) so that stages and their scales start on 16-byte
// boundaries; other K use the generic kernel.
bool qgemv_i8_fast_shape_ok(uint32_t rows, uint32_t k) {
    if (rows < 1 || rows > 8 || k < 512 || k % 512 != 0) return false;
    const size_t warps = rows <= 2 ? 4 : 8;
    return i8::BAR_BYTES + warps * 2 * i8::STAGE + (size_t)rows * k + (size_t)rows * (k / GROUP) * 4 + 4 * i8::PEND_ROWS * 4 <= 227 * 1024 - 1024;
}

cudaError_t launch_qgemv_i8_fast(const GemvArgs &a, int sm_count, bool pdl, cudaStream_t s) {
    switch (a.rows) {
        case 1: return i8::launch_m<1>(a, sm_count, pdl, s);
        case 2: return i8::launch_m<2>(a, sm_count, pdl, s);
        case 3: return i8::launch_m<3>(a, sm_count, pdl, s);
        case 4: return i8::launch_m<4>(a, sm_count, pdl, s);
        case 5: return i8::launch_m<5>(a, sm_count, pdl, s);
        case 6: return i8::launch_m<6>(a, sm_count, pdl, s);
        case 7: return i8::launch_m<7>(a, sm_count, pdl, s);
        case 8: return i8::launch_m<8>(a, sm_count, pdl, s);
        default: return cudaErrorInvalidValue;
    }
}

// The same for Int4 nibble planes (see the kernel): same shapes (qgemv_i8_fast_shape_ok).
cudaError_t launch_qgemv_i4_fast(const GemvArgs &a, int sm_count, bool pdl, cudaStream_t s) {
    switch (a.rows) {
        case 1: return i8::launch_m<1, false, true>(a, sm_count, pdl, s);
        case 2: return i8::launch_m<2, false, true>(a, sm_count, pdl, s);
        case 3: return i8::launch_m<3, false, true>(a, sm_count, pdl, s);
        case 4: return i8::launch_m<4, false, true>(a, sm_count, pdl, s);
        case 5: return i8::launch_m<5, false, true>(a, sm_count, pdl, s);
        case 6: return i8::launch_m<6, false, true>(a, sm_count, pdl, s);
        case 7: return i8::launch_m<7, false, true>(a, sm_count, pdl, s);
        case 8: return i8::launch_m<8, false, true>(a, sm_count, pdl, s);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace lb

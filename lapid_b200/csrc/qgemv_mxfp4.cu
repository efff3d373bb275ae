// Decode GEMV over MXFP4 blocks (ggml `block_mxfp4`, crates/lapid-quant/src/mxfp4.rs: 32 elements in 17 bytes --
// one e8m0 scale byte, then 16 bytes whose low nibbles are elements 0..15 and high nibbles elements 16..31;
// x = KV[nibble] * 2^(e - 128) with KV the doubled e2m1 values) with lapid-cpu's int8-activation arithmetic
// (crates/lapid-cpu/src/mxfp4.rs:38-58):
//
//     acc += d * da_g * f32(sum_32 qa * KV[q])          one activation group per weight block
//
// One warp per weight row; a lane takes every 32nd block of the row. Blocks are 17 bytes long, so they start on
// any byte boundary: the 16 nibble bytes are fetched as aligned 32-bit words and funnel-shifted into place. Four
// codes become four int8 KV values with three byte-permutes and three logic operations (mxfp4_kv4 in common.cuh: the
// four nibbles of a 16-bit half are used as the permute's selector as they are), multiplied with `dp4a` against the
// activation planes (served by L1/L2), whose bytes one more permute per word brings into the same element order.
// Two forms. When a weight row is a multiple of 16 bytes (K a multiple of 512) every warp streams its rows through a
// shared-memory double buffer with 16-byte `cp.async` copies: the copy of the next row is in flight while the current
// one is multiplied (one and two activation rows, K up to 8192: 4096 x 4096 at one row 7.6 against 9.2 us, 14336 x 4096
// 15.8 against 17.2 us). Other launches read the blocks straight from global memory. Either way the kernel is bound
// by the instructions that unpack a block (some 120 per 32 weights at one row), not by HBM (0.2-0.3 of its rate);
// from three rows on the launches go to the tensor-core kernel of qgemv_mxfp4_mma.cu.
#include "common.cuh"
#include "kernels.h"

namespace lb {
namespace mx {

constexpr int WARPS = 8;

// One 17-byte block at `b` (global or shared memory, any alignment) against activation group g of every row.
template <int M> __device__ __forceinline__ void block_dot(const uint8_t *b, const GemvArgs &p, uint32_t g, uint32_t k, uint32_t kg, float (&acc)[M]) {
    const float d = e8m0_half(*b);
    // the 16 nibble bytes b[1..16] from the aligned words around them
    const uintptr_t q0 = (uintptr_t)(b + 1);
    const uint32_t *wp = (const uint32_t *)(q0 & ~(uintptr_t)3);
    const uint32_t sh = (uint32_t)(q0 & 3) * 8;
    uint32_t raw[5];
#pragma unroll
    for (int i = 0; i < 4; i++) raw[i] = wp[i];
    raw[4] = sh ? wp[4] : 0u;  // (aligned blocks end with the fourth word: nothing is read behind them)
    // word i holds the codes of elements 4i..4i+3 (low nibbles) and 16+4i.. (high nibbles): q[2i] = KV of elements
    // (4i, 4i+16, 4i+1, 4i+17), q[2i+1] of (4i+2, 4i+18, 4i+3, 4i+19) as int8 (mxfp4_kv4)
    uint32_t q[8];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t w = __funnelshift_r(raw[i], raw[i + 1], sh);
        q[2 * i] = mxfp4_kv4(w);
        q[2 * i + 1] = mxfp4_kv4(w >> 16);
    }
#pragma unroll
    for (int r = 0; r < M; r++) {
        const uint4 *ap = (const uint4 *)(p.qa + (uint64_t)r * k + (uint64_t)g * GROUP);
        const uint4 a0 = __ldg(ap), a1 = __ldg(ap + 1);
        const float da = __ldg(p.da + (uint64_t)r * kg + g);
        const uint32_t al[4] = {a0.x, a0.y, a0.z, a0.w}, ah[4] = {a1.x, a1.y, a1.z, a1.w};
        int dp = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {  // the activations in the same element order
            dp = __dp4a((int)q[2 * i], (int)prmt(al[i], ah[i], 0x5140u), dp);
            dp = __dp4a((int)q[2 * i + 1], (int)prmt(al[i], ah[i], 0x7362u), dp);
        }
        acc[r] = fmaf(d * da, (float)dp, acc[r]);
    }
}

// KS warps share a row and split its blocks (matrices with few rows and a long K would otherwise leave most warp slots of
// an SM empty); their partial sums meet in shared memory and are added in warp order.
template <int M, int KS> __global__ void __launch_bounds__(WARPS * 32) qgemv_mxfp4_kernel(GemvArgs p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t k = p.k, kg = k / GROUP;
    if (p.ids) {
        // Expert-indexed launch (Kernel::MatMulId at decode sizes): grid row y is one (token, slot) pair
        const uint32_t pair = blockIdx.y, token = pair / p.id_r;
        const int32_t id = p.ids[pair];
        const bool bad = id < 0 || (uint32_t)id >= p.id_e;
        if (bad && p.status && threadIdx.x == 0) atomicOr(p.status, 128);
        p.w += bad ? 0 : (uint64_t)id * p.id_stride;
        p.qa += (uint64_t)token * k;
        p.da += (uint64_t)token * kg;
        p.out_off += (uint64_t)pair * p.n;
    }
    constexpr int RPC = WARPS / KS;  // rows of a CTA per pass
    const int wg = warp / KS, ks = warp % KS;
    __shared__ float part[KS > 1 ? WARPS * M : 1];
    for (uint32_t base = blockIdx.x * RPC; base < p.n; base += gridDim.x * RPC) {  // (the same number of passes for every warp of the CTA)
        const uint32_t row = base + wg, rrow = row < p.n ? row : p.n - 1;  // (a row past the end repeats the last one; not stored)
        float acc[M];
#pragma unroll
        for (int r = 0; r < M; r++) acc[r] = 0.0f;
        const uint8_t *wrow = p.w + (uint64_t)rrow * kg * MXFP4_BYTES;
        for (uint32_t g = lane + 32 * ks; g < kg; g += 32 * KS) block_dot<M>(wrow + (uint64_t)g * MXFP4_BYTES, p, g, k, kg, acc);
#pragma unroll
        for (int r = 0; r < M; r++) {
            float v = acc[r];
#pragma unroll
            for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if constexpr (KS > 1) {
                if (lane == 0) part[warp * M + r] = v;
            } else if (lane == 0 && row < p.n) {
                const uint32_t bt = r / p.m, i = r % p.m;
                if (p.extra && !p.epi.n) v += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)i * p.ex_s1 + (int64_t)row * p.ex_s2];
                p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)i * p.out_rs + row] = v;
            }
        }
        if constexpr (KS > 1) {
            __syncthreads();
            if (ks == 0 && lane < M && row < p.n) {
                const int r = lane;
                float v = part[warp * M + r];
#pragma unroll
                for (int s2 = 1; s2 < KS; s2++) v += part[(warp + s2) * M + r];
                const uint32_t bt = r / p.m, i = r % p.m;
                if (p.extra && !p.epi.n) v += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)i * p.ex_s1 + (int64_t)row * p.ex_s2];
                p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)i * p.out_rs + row] = v;
            }
            __syncthreads();  // the partial sums are read: the next pass may overwrite them
        }
    }
}

// K a multiple of 512 (weight rows are multiples of 16 bytes): the same arithmetic with every warp's rows streamed
// through its own double buffer in shared memory. The weights do not depend on the launch before this one, so the
// first row is requested before that launch's results are waited for.
template <int M> __global__ void __launch_bounds__(WARPS * 32) qgemv_mxfp4_staged_kernel(GemvArgs p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(16) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t k = p.k, kg = k / GROUP, rowb = kg * MXFP4_BYTES;
    const uint32_t slot = rowb + 16;  // (the aligned loads around a block's last nibble bytes may reach up to three bytes past the row)
    uint8_t *buf = smem + (size_t)warp * 2 * slot;
    if (p.ids) {
        // Expert-indexed launch (Kernel::MatMulId at decode sizes): grid row y is one (token, slot) pair; the ids may
        // come from the launch before this one
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const uint32_t pair = blockIdx.y, token = pair / p.id_r;
        const int32_t id = p.ids[pair];
        const bool bad = id < 0 || (uint32_t)id >= p.id_e;
        if (bad && p.status && threadIdx.x == 0) atomicOr(p.status, 128);
        p.w += bad ? 0 : (uint64_t)id * p.id_stride;
        p.qa += (uint64_t)token * k;
        p.da += (uint64_t)token * kg;
        p.out_off += (uint64_t)pair * p.n;
    }
    auto request = [&](uint32_t row, uint8_t *dst) {
        const uint8_t *src = p.w + (uint64_t)row * rowb;
        for (uint32_t c = lane; c < rowb / 16; c += 32)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst + 16 * c)), "l"(src + 16 * (size_t)c) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const uint32_t stride = gridDim.x * WARPS;
    uint32_t row = blockIdx.x * WARPS + warp;
    if (row < p.n) request(row, buf);
    if (!p.ids) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int cur = 0; row < p.n; row += stride, cur ^= 1) {
        if (row + stride < p.n) {
            request(row + stride, buf + (cur ^ 1) * slot);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();  // every lane's part of the row has landed
        float acc[M];
#pragma unroll
        for (int r = 0; r < M; r++) acc[r] = 0.0f;
        const uint8_t *wrow = buf + cur * slot;
        for (uint32_t g = lane; g < kg; g += 32) block_dot<M>(wrow + g * MXFP4_BYTES, p, g, k, kg, acc);
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
        __syncwarp();  // the buffer is refilled one iteration from now: every lane is done reading it
    }
}

static bool g_staged = true;  // (tests switch the staged form off to reach the other one at the same shapes)
static int g_k_split = 0;     // warps per row of the direct form: 0: chosen per launch; 1, 2, 4: forced
template <int M> static cudaError_t launch_m(const GemvArgs &a, uint32_t pairs, int sm_count, bool pdl, cudaStream_t stream) {
    const uint32_t want = (a.n + WARPS - 1) / WARPS;
    uint32_t cap = (uint32_t)sm_count * 8;
    if (pairs > 1) cap = cap / pairs > 0 ? cap / pairs : 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(want < cap ? want : cap, pairs);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    // rows of 16-byte multiples at 16-byte aligned addresses: the staged form, for one and two activation rows (beyond
    // that the `dp4a` work hides the loads anyway) and while at least three CTAs' buffers fit an SM
    // (4096 x 14336 at eight rows: 83 us staged with one CTA per SM, 45 us direct)
    const size_t smem = (size_t)WARPS * 2 * ((size_t)a.k / GROUP * MXFP4_BYTES + 16);
    const bool aligned = a.k % 512 == 0 && ((uintptr_t)a.w & 15) == 0 && (!a.ids || (a.id_stride & 15) == 0);
    if (aligned && M <= 2 && smem <= 72 * 1024 && g_staged) {
        static DynamicSmemOptIn optin;
        cudaError_t e = optin.raise((const void *)qgemv_mxfp4_staged_kernel<M>, smem);
        if (e != cudaSuccess) return e;
        cfg.dynamicSmemBytes = smem;
        return cudaLaunchKernelEx(&cfg, qgemv_mxfp4_staged_kernel<M>, a);
    }
    // direct loads: one warp per row, or two / four warps per row when the rows alone leave most warp slots empty
    // and are long enough to split
    const uint64_t rows = (uint64_t)a.n * pairs, slots = (uint64_t)sm_count * 32, steps = a.k / GROUP / 32;
    int ksp = 1;
    if (g_k_split) ksp = g_k_split;
    else
        while (ksp < 4 && rows * ksp < slots && steps / (2 * ksp) >= 2) ksp *= 2;
    if (ksp > 1) {
        const uint32_t rpc = WARPS / ksp, want2 = (a.n + rpc - 1) / rpc;
        cfg.gridDim = dim3(want2 < cap ? want2 : cap, pairs);
        if (ksp == 2) return cudaLaunchKernelEx(&cfg, qgemv_mxfp4_kernel<M, 2>, a);
        return cudaLaunchKernelEx(&cfg, qgemv_mxfp4_kernel<M, 4>, a);
    }
    return cudaLaunchKernelEx(&cfg, qgemv_mxfp4_kernel<M, 1>, a);
}

}  // namespace mx

void qgemv_mxfp4_set_staged(int on) { mx::g_staged = on != 0; }
void qgemv_mxfp4_set_k_split(int ways) { mx::g_k_split = ways == 1 || ways == 2 || ways == 4 ? ways : 0; }

cudaError_t launch_qgemv_mxfp4(const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream) {
    if (args.n == 0 || args.rows == 0) return cudaSuccess;
    if (args.k % GROUP != 0 || ((uintptr_t)args.w & 3) != 0) return cudaErrorInvalidValue;
    if (args.ids) {  // one-row GEMV per (token, slot) pair
        if (args.id_r == 0 || args.id_e == 0 || args.rows > 8 || (uint64_t)args.rows * args.id_r > 65535 || (args.id_stride & 3))
            return cudaErrorInvalidValue;
        GemvArgs one = args;
        one.rows = 1;
        one.m = 1;
        return mx::launch_m<1>(one, args.rows * args.id_r, sm_count, pdl, stream);
    }
    switch (args.rows) {
        case 1: return mx::launch_m<1>(args, 1, sm_count, pdl, stream);
        case 2: return mx::launch_m<2>(args, 1, sm_count, pdl, stream);
        case 3: return mx::launch_m<3>(args, 1, sm_count, pdl, stream);
        case 4: return mx::launch_m<4>(args, 1, sm_count, pdl, stream);
        case 5: return mx::launch_m<5>(args, 1, sm_count, pdl, stream);
        case 6: return mx::launch_m<6>(args, 1, sm_count, pdl, stream);
        case 7: return mx::launch_m<7>(args, 1, sm_count, pdl, stream);
        case 8: return mx::launch_m<8>(args, 1, sm_count, pdl, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace lb

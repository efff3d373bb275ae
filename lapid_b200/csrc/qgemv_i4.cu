// Decode GEMV over Int4 nibble planes (lapid's `int4`: byte j of a 32-element group holds element j in
// its low and element j + 16 in its high nibble, x = (q - 8) * d, one f16 scale per group;
// crates/lapid-quant/src/lib.rs:10-17), with lapid-cpu's int8-activation arithmetic
// (crates/lapid-cpu/src/matmul/qkernels.rs:60-84 over QMat::group_i8, crates/lapid-cpu/src/qmat.rs:97-112):
//
//     acc += f32(sum_32 qa * (q - 8)) * (da_g * db_g)
//
// One warp per weight row: a lane takes every 32nd group of the row with one 128-bit load (16 bytes =
// one group), re-centres the nibbles to signed bytes with two masks and two byte-wise subtractions and
// multiplies them with `dp4a` against the activation planes (served by L1/L2). A straightforward
// streaming kernel: the format is outside the benchmark's configurations and has no bulk-copy or
// tensor-core variant yet.
#include "common.cuh"
#include "kernels.h"

namespace lb {
namespace i4 {

constexpr int WARPS = 8;

template <int M> __global__ void __launch_bounds__(WARPS * 32) qgemv_i4_kernel(GemvArgs p) {
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
    const uint16_t *scales = (const uint16_t *)(p.w + p.scales_offset);
    for (uint32_t row = blockIdx.x * WARPS + warp; row < p.n; row += gridDim.x * WARPS) {
        float acc[M];
#pragma unroll
        for (int r = 0; r < M; r++) acc[r] = 0.0f;
        const uint4 *wrow = (const uint4 *)(p.w + (uint64_t)row * (k / 2));
#pragma unroll 2
        for (uint32_t g = lane; g < kg; g += 32) {
            const uint4 v = __ldg(wrow + g);
            const float db = half_bits_to_float(__ldg(scales + (uint64_t)row * kg + g));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t lo[4], hi[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                lo[i] = __vsub4(w[i] & 0x0F0F0F0Fu, 0x08080808u);         // elements 4i .. 4i+3
                hi[i] = __vsub4((w[i] >> 4) & 0x0F0F0F0Fu, 0x08080808u);  // elements 16 + 4i ..
            }
#pragma unroll
            for (int r = 0; r < M; r++) {
                const uint4 *ap = (const uint4 *)(p.qa + (uint64_t)r * k + (uint64_t)g * GROUP);
                const uint4 a0 = __ldg(ap), a1 = __ldg(ap + 1);
                const float da = __ldg(p.da + (uint64_t)r * kg + g);
                int d = __dp4a((int)lo[0], (int)a0.x, 0);
                d = __dp4a((int)lo[1], (int)a0.y, d);
                d = __dp4a((int)lo[2], (int)a0.z, d);
                d = __dp4a((int)lo[3], (int)a0.w, d);
                d = __dp4a((int)hi[0], (int)a1.x, d);
                d = __dp4a((int)hi[1], (int)a1.y, d);
                d = __dp4a((int)hi[2], (int)a1.z, d);
                d = __dp4a((int)hi[3], (int)a1.w, d);
                acc[r] = fmaf((float)d, da * db, acc[r]);
            }
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
}

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
    return cudaLaunchKernelEx(&cfg, qgemv_i4_kernel<M>, a);
}

}  // namespace i4

cudaError_t launch_qgemv_i4(const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream) {
    if (args.n == 0 || args.rows == 0) return cudaSuccess;
    if (args.k % GROUP != 0 || ((uintptr_t)args.w & 15) != 0 || (args.k / 2) % 16 != 0) return cudaErrorInvalidValue;
    if (args.ids) {  // one-row GEMV per (token, slot) pair
        if (args.id_r == 0 || args.id_e == 0 || args.rows > 8 || (uint64_t)args.rows * args.id_r > 65535 || (args.id_stride & 15))
            return cudaErrorInvalidValue;
        GemvArgs one = args;
        one.rows = 1;
        one.m = 1;
        return i4::launch_m<1>(one, args.rows * args.id_r, sm_count, pdl, stream);
    }
    switch (args.rows) {
        case 1: return i4::launch_m<1>(args, 1, sm_count, pdl, stream);
        case 2: return i4::launch_m<2>(args, 1, sm_count, pdl, stream);
        case 3: return i4::launch_m<3>(args, 1, sm_count, pdl, stream);
        case 4: return i4::launch_m<4>(args, 1, sm_count, pdl, stream);
        case 5: return i4::launch_m<5>(args, 1, sm_count, pdl, stream);
        case 6: return i4::launch_m<6>(args, 1, sm_count, pdl, stream);
        case 7: return i4::launch_m<7>(args, 1, sm_count, pdl, stream);
        case 8: return i4::launch_m<8>(args, 1, sm_count, pdl, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace lb

// Decode GEMV over ggml's grid-based i-quants (IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS; see iquant.cuh for the block
// layouts) with lapid-cpu's int8-activation arithmetic (crates/lapid-cpu/src/iquant.rs:92-128):
//
//     acc += sc[h] * da[h / 2] * f32(sum_16 qa * grid * sign)        per 16-element half h of a block
//
// These formats hold 2 to 3 bits per weight, so a launch reads little from HBM and spends its time looking up
// grid entries: the kernel is built around that. Each CTA first copies the format's codebook (1 to 8 KB) into
// shared memory. One warp takes one weight row at a time; a lane takes one half (two 8-groups) of a block, so a
// warp covers two blocks per step: it reads the half's index and sign bits straight from the 2-byte-aligned block
// (L1 serves the neighbours), fetches the two grid entries from shared memory, applies the signs to get sixteen
// int8 weights in four registers, and multiplies them with `dp4a` against each activation row's sixteen int8
// values (one 16-byte load per row from the activation planes). The sum over 16 elements is exact, the products
// are the reference's; only the order in which the halves are added differs (lanes, then a shuffle tree).
#include "common.cuh"
#include "iquant.cuh"
#include "kernels.h"

namespace lb {
namespace iq {

constexpr int WARPS = 8;

template <int FMT, int M> __global__ void __launch_bounds__(WARPS * 32) qgemv_iq_kernel(GemvArgs p, const uint8_t *__restrict__ grid_global) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ __align__(16) uint8_t grid[iq_grid_bytes(FMT)];
    {  // the codebook never changes: it may be read before the launch this one depends on has finished
        const uint4 *src = (const uint4 *)grid_global;
        uint4 *dst = (uint4 *)grid;
        for (int i = threadIdx.x; i < iq_grid_bytes(FMT) / 16; i += WARPS * 32) dst[i] = __ldg(src + i);
    }
    __syncthreads();
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t k = p.k, kg = k / GROUP, nblk = k / QK;
    constexpr int BB = iq_block_bytes(FMT);
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
    const int h = lane & 15;  // this lane's half of the block
    for (uint32_t row = blockIdx.x * WARPS + warp; row < p.n; row += gridDim.x * WARPS) {
        float acc[M];
#pragma unroll
        for (int r = 0; r < M; r++) acc[r] = 0.0f;
        const uint8_t *wrow = p.w + (uint64_t)row * nblk * BB;
        for (uint32_t blk = lane >> 4; blk < nblk; blk += 2) {
            const uint8_t *b = wrow + (uint64_t)blk * BB;
            uint32_t w[4], s0, s1;
            iq_group8<FMT>(b, 2 * h, grid, w[0], w[1], s0);
            iq_group8<FMT>(b, 2 * h + 1, grid, w[2], w[3], s1);
            w[0] = iq_apply_signs(w[0], s0);
            w[1] = iq_apply_signs(w[1], s0 >> 4);
            w[2] = iq_apply_signs(w[2], s1);
            w[3] = iq_apply_signs(w[3], s1 >> 4);
            const float sc = iq_half_scale<FMT>(b, h);
            const uint32_t g = blk * 8 + (h >> 1);  // activation group of this half
#pragma unroll
            for (int r = 0; r < M; r++) {
                const uint4 a = __ldg((const uint4 *)(p.qa + (uint64_t)r * k + (uint64_t)blk * QK + 16 * h));
                const float da = __ldg(p.da + (uint64_t)r * kg + g);
                int dot = __dp4a((int)w[0], (int)a.x, 0);
                dot = __dp4a((int)w[1], (int)a.y, dot);
                dot = __dp4a((int)w[2], (int)a.z, dot);
                dot = __dp4a((int)w[3], (int)a.w, dot);
                acc[r] += (sc * da) * (float)dot;
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

template <int FMT, int M> static cudaError_t launch_m(const GemvArgs &a, const uint8_t *grid, uint32_t pairs, int sm_count, bool pdl, cudaStream_t stream) {
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
    return cudaLaunchKernelEx(&cfg, qgemv_iq_kernel<FMT, M>, a, grid);
}

template <int FMT> static cudaError_t launch_fmt(const GemvArgs &args, const uint8_t *grid, int sm_count, bool pdl, cudaStream_t stream) {
    if (args.ids) {  // one-row GEMV per (token, slot) pair
        if (args.id_r == 0 || args.id_e == 0 || args.rows > 8 || (uint64_t)args.rows * args.id_r > 65535 || (args.id_stride & 1))
            return cudaErrorInvalidValue;
        GemvArgs one = args;
        one.rows = 1;
        one.m = 1;
        return launch_m<FMT, 1>(one, grid, args.rows * args.id_r, sm_count, pdl, stream);
    }
    switch (args.rows) {
        case 1: return launch_m<FMT, 1>(args, grid, 1, sm_count, pdl, stream);
        case 2: return launch_m<FMT, 2>(args, grid, 1, sm_count, pdl, stream);
        case 3: return launch_m<FMT, 3>(args, grid, 1, sm_count, pdl, stream);
        case 4: return launch_m<FMT, 4>(args, grid, 1, sm_count, pdl, stream);
        case 5: return launch_m<FMT, 5>(args, grid, 1, sm_count, pdl, stream);
        case 6: return launch_m<FMT, 6>(args, grid, 1, sm_count, pdl, stream);
        case 7: return launch_m<FMT, 7>(args, grid, 1, sm_count, pdl, stream);
        case 8: return launch_m<FMT, 8>(args, grid, 1, sm_count, pdl, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace iq

cudaError_t launch_qgemv_iq(int fmt, const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream) {
    if (args.n == 0 || args.rows == 0) return cudaSuccess;
    if (!is_iq(fmt) || args.k % QK != 0 || ((uintptr_t)args.w & 1) != 0 || ((uintptr_t)args.qa & 15) != 0) return cudaErrorInvalidValue;
    const uint8_t *grids = iq_grids();
    if (!grids) return cudaErrorNotReady;
    const uint8_t *grid = grids + iq_grid_offset(fmt);
    switch (fmt) {
        case FMT_IQ2XXS: return iq::launch_fmt<FMT_IQ2XXS>(args, grid, sm_count, pdl, stream);
        case FMT_IQ2XS: return iq::launch_fmt<FMT_IQ2XS>(args, grid, sm_count, pdl, stream);
        case FMT_IQ2S: return iq::launch_fmt<FMT_IQ2S>(args, grid, sm_count, pdl, stream);
        default: return iq::launch_fmt<FMT_IQ3XXS>(args, grid, sm_count, pdl, stream);
    }
}

}  // namespace lb

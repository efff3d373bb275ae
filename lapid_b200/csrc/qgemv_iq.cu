// Decode GEMV over ggml's grid-based i-quants (IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS; see iquant.cuh for the block
// layouts) with lapid-cpu's int8-activation arithmetic (crates/lapid-cpu/src/iquant.rs:92-128):
//
//     acc += sc[h] * da[h / 2] * f32(sum_16 qa * grid * sign)        per 16-element half h of a block
//
// These formats hold 2 to 3 bits per weight, so a launch reads little from HBM and spends its time looking up
// grid entries and applying signs: the kernel is built around that. Each CTA first copies the format's codebook (1 to
// 8 KB) into shared memory; a lookup is one shared-memory load at a data-dependent address (bank conflicts are the
// cost that remains), the signs are applied in three arithmetic instructions per four weights (signed4 below) rather
// than through a second table.
// One warp takes ROWS (1 or 2) weight rows at a time; a lane takes one 32-element sub-block of a block (four 8-groups: 4 to
// 12 bytes of indices and signs, read as 16-bit halves because blocks are only 2-byte aligned), so a warp covers
// four blocks per step. The lane turns its sub-block into eight registers of int8 weights and multiplies them with
// `dp4a` against each activation row's 32 int8 values (two 16-byte loads per row from the activation planes, shared
// by the ROWS weight rows). The sums over 16 elements are exact and the products are the reference's; only the
// order in which the halves are added differs (lanes, then a shuffle tree).
#include "common.cuh"
#include "iquant.cuh"
#include "kernels.h"

namespace lb {
namespace iq {

// Four grid bytes with the signs of bits 0..3 of `s4` (0..15) applied, as four int8 values. The multiplication puts
// sign bit j into the top bit of byte j (the other product bits land elsewhere), the byte-permute in its
// sign-replicating mode turns that into the byte mask m, and (g ^ m) + (m & 0x01010101) negates the masked bytes:
// a grid byte is never 0, so the + 1 of a negation never carries into the next byte.
__device__ __forceinline__ uint32_t signed4(uint32_t g, uint32_t s4) {
    uint32_t m;  // prmt's selector nibbles 8 | j: replicate the top bit of byte j (the __byte_perm intrinsic drops that bit)
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(m) : "r"(s4 * 0x10204080u), "r"(0u), "r"(0xBA98u));
    return (g ^ m) + (m & 0x01010101u);
}
// ... and of the 8-group whose sign bits are `s8`: lo takes bits 0..3, hi bits 4..7
__device__ __forceinline__ void signed8(uint32_t glo, uint32_t ghi, uint32_t s8, uint32_t &lo, uint32_t &hi) {
    lo = signed4(glo, s8 & 15u);
    hi = signed4(ghi, s8 >> 4);
}

// The eight int8-weight registers (w[2l], w[2l + 1] = 8-group l) and the two half scales of sub-block ib.
template <int FMT>
__device__ __forceinline__ void unpack32(const uint8_t *b, int ib, const uint8_t *grid, uint32_t (&w)[8], float &sc0, float &sc1) {
    const float d = half_bits_to_float(ld16(b));
    uint32_t idx[4], sg[4], s0, s1;  // grid entry and sign-table entry of each 8-group; the 4-bit scales
    if constexpr (FMT == FMT_IQ2XXS) {
        const uint8_t *p = b + 2 + 8 * ib;
        const uint32_t q = ld32_by16(p), a1 = ld32_by16(p + 4);
#pragma unroll
        for (int l = 0; l < 4; l++) idx[l] = (q >> (8 * l)) & 255u, sg[l] = (a1 >> (7 * l)) & 127u;
        s0 = s1 = a1 >> 28;
    } else if constexpr (FMT == FMT_IQ2XS) {
        const uint8_t *p = b + 2 + 8 * ib;
        const uint32_t q01 = ld32_by16(p), q23 = ld32_by16(p + 4), sc = b[66 + ib];
        idx[0] = q01 & 511u, sg[0] = (q01 >> 9) & 127u, idx[1] = (q01 >> 16) & 511u, sg[1] = q01 >> 25;
        idx[2] = q23 & 511u, sg[2] = (q23 >> 9) & 127u, idx[3] = (q23 >> 16) & 511u, sg[3] = q23 >> 25;
        s0 = sc & 15u, s1 = sc >> 4;
    } else if constexpr (FMT == FMT_IQ2S) {
        const uint32_t q = ld32_by16(b + 2 + 4 * ib), sn = ld32_by16(b + 34 + 4 * ib), qh = b[66 + ib], sc = b[74 + ib];
#pragma unroll
        for (int l = 0; l < 4; l++) idx[l] = ((q >> (8 * l)) & 255u) | (((qh >> (2 * l)) & 3u) << 8), sg[l] = (sn >> (8 * l)) & 255u;
        s0 = sc & 15u, s1 = sc >> 4;
    } else {
        const uint32_t aux = ld32_by16(b + 66 + 4 * ib);
#pragma unroll
        for (int l = 0; l < 4; l++) sg[l] = (aux >> (7 * l)) & 127u;
        s0 = s1 = aux >> 28;
    }
    if constexpr (FMT == FMT_IQ3XXS) {
        const uint8_t *p = b + 2 + 8 * ib;
        const uint32_t q0 = ld32_by16(p), q1 = ld32_by16(p + 4);
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t q = l < 2 ? q0 >> (16 * l) : q1 >> (16 * (l - 2));
            signed8(*(const uint32_t *)(grid + 4 * (q & 255u)), *(const uint32_t *)(grid + 4 * ((q >> 8) & 255u)), iq_ksign(sg[l]), w[2 * l], w[2 * l + 1]);
        }
    } else {
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint2 g = *(const uint2 *)(grid + 8 * idx[l]);
            signed8(g.x, g.y, FMT == FMT_IQ2S ? sg[l] : iq_ksign(sg[l]), w[2 * l], w[2 * l + 1]);
        }
    }
    constexpr float F = FMT == FMT_IQ3XXS ? 0.5f : 0.25f;  // crates/lapid-cpu/src/iquant.rs:66-89, each operation rounded on its own
    sc0 = xmul(xmul(d, xadd(0.5f, (float)s0)), F);
    sc1 = xmul(xmul(d, xadd(0.5f, (float)s1)), F);
}

// KS warps share the rows of a warp group and split their blocks (matrices with few rows and a long K would otherwise
// leave most warp slots of an SM empty); their partial sums meet in shared memory and are added in warp order.
template <int FMT, int M, int ROWS, int WARPS, int KS>
__global__ void __launch_bounds__(WARPS * 32) qgemv_iq_kernel(GemvArgs p, const uint8_t *__restrict__ grid_global) {
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
    const int ib = lane & 7;  // this lane's sub-block
    constexpr int RPC = WARPS / KS * ROWS;  // rows of a CTA per pass
    const int wg = warp / KS, ks = warp % KS;
    __shared__ float part[KS > 1 ? WARPS * ROWS * M : 1];
    for (uint32_t base = blockIdx.x * RPC; base < p.n; base += gridDim.x * RPC) {  // (the same number of passes for every warp of the CTA)
        const uint32_t row0 = base + wg * ROWS;
        float acc[ROWS][M];
#pragma unroll
        for (int j = 0; j < ROWS; j++)
#pragma unroll
            for (int r = 0; r < M; r++) acc[j][r] = 0.0f;
        for (uint32_t blk = (lane >> 3) + 4 * ks; blk < nblk; blk += 4 * KS) {
            uint32_t w[ROWS][8];
            float sc[ROWS][2];
#pragma unroll
            for (int j = 0; j < ROWS; j++) {
                const uint32_t row = row0 + j < p.n ? row0 + j : p.n - 1;  // (a row past the end repeats the last one; not stored)
                unpack32<FMT>(p.w + ((uint64_t)row * nblk + blk) * BB, ib, grid, w[j], sc[j][0], sc[j][1]);
            }
            const uint32_t g = blk * 8 + ib;  // activation group of this sub-block
#pragma unroll
            for (int r = 0; r < M; r++) {
                const uint4 *ap = (const uint4 *)(p.qa + (uint64_t)r * k + (uint64_t)g * GROUP);
                const uint4 a0 = __ldg(ap), a1 = __ldg(ap + 1);
                const float da = __ldg(p.da + (uint64_t)r * kg + g);
#pragma unroll
                for (int j = 0; j < ROWS; j++) {
                    int d0 = __dp4a((int)w[j][0], (int)a0.x, 0);
                    d0 = __dp4a((int)w[j][1], (int)a0.y, d0);
                    d0 = __dp4a((int)w[j][2], (int)a0.z, d0);
                    d0 = __dp4a((int)w[j][3], (int)a0.w, d0);
                    int d1 = __dp4a((int)w[j][4], (int)a1.x, 0);
                    d1 = __dp4a((int)w[j][5], (int)a1.y, d1);
                    d1 = __dp4a((int)w[j][6], (int)a1.z, d1);
                    d1 = __dp4a((int)w[j][7], (int)a1.w, d1);
                    acc[j][r] += (sc[j][0] * da) * (float)d0;
                    acc[j][r] += (sc[j][1] * da) * (float)d1;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < ROWS; j++) {
#pragma unroll
            for (int r = 0; r < M; r++) {
                float v = acc[j][r];
#pragma unroll
                for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                const uint32_t row = row0 + j;
                if constexpr (KS > 1) {
                    if (lane == 0) part[(warp * ROWS + j) * M + r] = v;
                } else if (lane == 0 && row < p.n) {
                    const uint32_t bt = r / p.m, i = r % p.m;
                    if (p.extra && !p.epi.n) v += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)i * p.ex_s1 + (int64_t)row * p.ex_s2];
                    p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)i * p.out_rs + row] = v;
                }
            }
        }
        if constexpr (KS > 1) {
            __syncthreads();
            if (ks == 0 && lane < ROWS * M) {  // one lane per (row, activation row) of the group
                const int j = lane / M, r = lane % M;
                float v = part[(warp * ROWS + j) * M + r];
#pragma unroll
                for (int s2 = 1; s2 < KS; s2++) v += part[((warp + s2) * ROWS + j) * M + r];
                const uint32_t row = row0 + j;
                if (row < p.n) {
                    const uint32_t bt = r / p.m, i = r % p.m;
                    if (p.extra && !p.epi.n) v += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)i * p.ex_s1 + (int64_t)row * p.ex_s2];
                    p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)i * p.out_rs + row] = v;
                }
            }
            __syncthreads();  // the partial sums are read: the next pass may overwrite them
        }
    }
}

template <int FMT, int M, int ROWS, int WARPS, int KS = 1> static cudaError_t launch_r(const GemvArgs &a, const uint8_t *grid, uint32_t pairs, int sm_count, bool pdl, cudaStream_t stream) {
    constexpr uint32_t RPC = WARPS / KS * ROWS;
    const uint32_t want = (a.n + RPC - 1) / RPC;
    uint32_t cap = (uint32_t)sm_count * 8 * (8 / WARPS);
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
    return cudaLaunchKernelEx(&cfg, qgemv_iq_kernel<FMT, M, ROWS, WARPS, KS>, a, grid);
}

// Two weight rows per warp share the activation loads and give the scheduler two independent decode chains: the
// fastest form measured where the matrix has rows enough to fill the SMs' warp slots that way (four rows per warp need
// 128 registers and lose more to occupancy than they save in loads). With fewer rows: one row per warp, and two or
// four warps per row when even that leaves slots empty and the rows are long enough to split (4096 x 14336 at one
// activation row: 24.2 us with two rows per warp, 19.8 with one).
static int g_rows_per_warp = 0;  // 0: chosen per launch; 1, 2: forced (tests, sweeps)
static int g_k_split = 0;        // 0: chosen per launch; 1, 2, 4: forced
template <int FMT, int M> static cudaError_t launch_m(const GemvArgs &a, const uint8_t *grid, uint32_t pairs, int sm_count, bool pdl, cudaStream_t stream) {
    const uint64_t slots = (uint64_t)sm_count * 32;  // warps that keep the SMs' schedulers busy
    const uint64_t rows = (uint64_t)a.n * pairs, steps = a.k / QK / 4;  // steps: passes of a warp over a row at four blocks per pass
    int rpw = g_rows_per_warp ? g_rows_per_warp : ((rows + 1) / 2 >= slots ? 2 : 1);
    int ksp = 1;
    if (g_k_split) ksp = g_k_split;
    else if (rpw == 1)
        while (ksp < 4 && rows * ksp < slots && steps / (2 * ksp) >= 2) ksp *= 2;
    if (rpw == 2) return launch_r<FMT, M, 2, 4>(a, grid, pairs, sm_count, pdl, stream);
    if (ksp == 2) return launch_r<FMT, M, 1, 8, 2>(a, grid, pairs, sm_count, pdl, stream);
    if (ksp == 4) return launch_r<FMT, M, 1, 8, 4>(a, grid, pairs, sm_count, pdl, stream);
    return launch_r<FMT, M, 1, 8>(a, grid, pairs, sm_count, pdl, stream);
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

void qgemv_iq_set_rows_per_warp(int rows) { iq::g_rows_per_warp = rows == 1 || rows == 2 ? rows : 0; }
void qgemv_iq_set_k_split(int ways) { iq::g_k_split = ways == 1 || ways == 2 || ways == 4 ? ways : 0; }

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

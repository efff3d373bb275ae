// Routing for Kernel::MatMulId (crates/lapid-compiler/src/ir.rs:425-443) above decode sizes:
// out[t, s, :] = W[ids[t, s]] x[t] for t tokens, r slots each, over a stack of e expert matrices.
// lapid-cpu groups the (token, slot) pairs by expert on the host and runs one matmul per used
// expert (crates/lapid-cpu/src/moe.rs:40-120). Here the grouping happens on the device, so the
// launch needs no host round trip and can be captured in a graph:
//
//   route   one CTA counts the pairs of every expert, gives every expert a run of whole
//           activation tiles (`mt` rows each; the run's last tile is padded), and writes
//             tile_expert[tile]  the expert whose matrix the tile multiplies, -1 past the last used tile
//             row_pair[row]      the pair that sits in this row of the tile space, -1 for padding
//   GEMM    the ordinary tiled kernels (tensor-core or exact f32) over the tile space: a CTA
//           looks up its tile's expert, exits when there is none, reads activation row
//           row_pair[row] / r and stores to output row row_pair[row]
//
// The number of used tiles is only known on the device; the grid covers the upper bound
// pairs / mt + min(e, pairs). Which row of an expert's run a pair lands in depends on the order
// of the atomic increments, but every output row is computed independently of the other rows of
// its tile, so the result does not. An id outside [0, e) sets bit 128 of the status word; its
// pair is left out (the host reports index_out_of_range, as the reference does before running).
#include <cuda_bf16.h>

#include "common.cuh"
#include "kernels.h"

namespace lb {

constexpr int ROUTE_THREADS = 1024;

__global__ void __launch_bounds__(ROUTE_THREADS) moe_route_kernel(MoeRouteArgs a) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ uint32_t warp_sum[ROUTE_THREADS / 32];
    __shared__ uint32_t base_tile;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (uint32_t x = tid; x < a.experts; x += ROUTE_THREADS) a.counts[x] = 0, a.cursor[x] = 0;
    for (uint32_t i = tid; i < a.max_tiles; i += ROUTE_THREADS) a.tile_expert[i] = -1;
    for (uint32_t i = tid; i < a.max_tiles * a.mt; i += ROUTE_THREADS) a.row_pair[i] = -1;
    if (tid == 0) base_tile = 0;
    __syncthreads();
    bool bad = false;
    for (uint32_t p = tid; p < a.pairs; p += ROUTE_THREADS) {
        const int32_t id = a.ids[p];
        if (id < 0 || (uint32_t)id >= a.experts) bad = true;
        else atomicAdd(&a.counts[id], 1);
    }
    if (bad && a.status) atomicOr(a.status, 128);
    __syncthreads();
    // exclusive scan of the experts' tile counts, ROUTE_THREADS experts at a time
    for (uint32_t x0 = 0; x0 < a.experts; x0 += ROUTE_THREADS) {
        const uint32_t x = x0 + tid;
        const uint32_t tiles = x < a.experts ? ((uint32_t)a.counts[x] + a.mt - 1) / a.mt : 0;
        uint32_t inc = tiles;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, inc, o);
            if ((int)lane >= o) inc += v;
        }
        if (lane == 31) warp_sum[warp] = inc;
        __syncthreads();
        uint32_t before = base_tile;
        for (uint32_t w = 0; w < warp; w++) before += warp_sum[w];
        const uint32_t first = before + inc - tiles;
        if (x < a.experts) {
            a.offsets[x] = (int32_t)(first * a.mt);
            for (uint32_t i = 0; i < tiles && first + i < a.max_tiles; i++) a.tile_expert[first + i] = (int32_t)x;
        }
        __syncthreads();
        if (tid == ROUTE_THREADS - 1) base_tile = before + inc;
        __syncthreads();
    }
    for (uint32_t p = tid; p < a.pairs; p += ROUTE_THREADS) {
        const int32_t id = a.ids[p];
        if (id < 0 || (uint32_t)id >= a.experts) continue;
        const uint32_t pos = (uint32_t)a.offsets[id] + (uint32_t)atomicAdd(&a.cursor[id], 1);
        if (pos < a.max_tiles * a.mt) a.row_pair[pos] = (int32_t)p;
    }
}

// bf16 copy of the activation rows in tile-space order (the tensor-core kernel's A operand):
// row i of dst = x[row_pair[i] / r], zeros for a padding row. blockIdx.y walks the rows.
__global__ void __launch_bounds__(256) moe_gather_bf16_kernel(const float *x, const int32_t *row_pair, uint32_t r, uint32_t k,
                                                              uint32_t rows, __nv_bfloat16 *dst) {
    for (uint32_t row = blockIdx.y; row < rows; row += gridDim.y) {
        const int32_t pair = row_pair[row];
        uint4 *out = (uint4 *)(dst + (size_t)row * k);
        const float4 *src = pair < 0 ? nullptr : (const float4 *)(x + (size_t)((uint32_t)pair / r) * k);
        for (uint32_t c8 = blockIdx.x * blockDim.x + threadIdx.x; c8 < k / 8; c8 += gridDim.x * blockDim.x) {
            __nv_bfloat162 o[4];
            if (src) {
                const float4 lo = src[2 * c8], hi = src[2 * c8 + 1];
                o[0] = __floats2bfloat162_rn(lo.x, lo.y);
                o[1] = __floats2bfloat162_rn(lo.z, lo.w);
                o[2] = __floats2bfloat162_rn(hi.x, hi.y);
                o[3] = __floats2bfloat162_rn(hi.z, hi.w);
            } else {
                o[0] = o[1] = o[2] = o[3] = __floats2bfloat162_rn(0.0f, 0.0f);
            }
            out[c8] = *(const uint4 *)o;
        }
    }
}

uint32_t moe_max_tiles(uint64_t pairs, uint64_t experts, uint32_t mt) {
    return (uint32_t)(pairs / mt + (experts < pairs ? experts : pairs));
}

// counts, cursor, offsets (experts each), tile_expert, row_pair: 4-byte integers, 256-byte aligned as a whole
size_t moe_route_bytes(uint64_t pairs, uint64_t experts, uint32_t mt) {
    const uint64_t tiles = moe_max_tiles(pairs, experts, mt);
    return (size_t)((4 * (3 * experts + tiles + tiles * mt) + 255) & ~(uint64_t)255);
}

void moe_route_layout(void *scratch, uint64_t pairs, uint64_t experts, uint32_t mt, MoeRouteArgs &a) {
    int32_t *p = (int32_t *)scratch;
    a.pairs = (uint32_t)pairs;
    a.experts = (uint32_t)experts;
    a.mt = mt;
    a.max_tiles = moe_max_tiles(pairs, experts, mt);
    a.counts = p;
    a.cursor = p + experts;
    a.offsets = p + 2 * experts;
    a.tile_expert = p + 3 * experts;
    a.row_pair = a.tile_expert + a.max_tiles;
}

cudaError_t launch_moe_route(const MoeRouteArgs &a, bool pdl, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(ROUTE_THREADS);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, moe_route_kernel, a);
}

cudaError_t launch_moe_gather_bf16(const float *x, const MoeRouteArgs &a, uint32_t r, uint32_t k, void *dst, cudaStream_t stream) {
    const uint32_t rows = a.max_tiles * a.mt;
    if (rows == 0) return cudaSuccess;
    if (k % 8 != 0 || ((uintptr_t)x & 15) != 0) return cudaErrorInvalidValue;
    const dim3 grid((k / 8 + 255) / 256, rows < 65535u ? rows : 65535u);
    moe_gather_bf16_kernel<<<grid, 256, 0, stream>>>(x, a.row_pair, r, k, rows, (__nv_bfloat16 *)dst);
    return cudaGetLastError();
}

}  // namespace lb

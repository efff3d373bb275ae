// One-shot all-reduce (f32 sum, in place) of a row-parallel projection's partial results over the
// GPUs of one NVLink/NVSwitch domain, through peer-mapped memory. The reference has no multi-GPU
// code; this replaces a library all-reduce whose latency (tens of microseconds per call inside a
// token that needs two calls per layer) dominates tensor-parallel decode.
//
// Every rank owns one "symmetric" buffer, mapped into every peer's address space:
//     [0, 256)      flags[src]   u32: the epoch src has finished pushing
//     [256, 512)    epoch, done  u32: this rank's call counter and its CTA-completion counter
//     [512, ...)    slots[parity][src][max_elems]  f32
// One kernel per call, no grid-wide barrier:
//   push    each CTA stores its chunk of the local partial into slot[rank] of EVERY rank's buffer
//           (plain peer stores over NVLink; 32 KB per peer at decode sizes), fences at system scope
//           and counts itself done; the last CTA of the rank publishes the new epoch in every
//           rank's flags[rank] with a release store
//   wait    every CTA acquires all `world` flags of its own buffer (bounded spin)
//   reduce  each CTA sums its chunk of the `world` slots in rank order and writes the result over
//           the local partial: all ranks add the same numbers in the same order, so the result is
//           bit-identical everywhere and independent of timing
// Slots are double-buffered by epoch parity: a rank can be at most one call ahead of a peer (its
// next call cannot pass its own wait before the peer has pushed), so it never overwrites a slot a
// peer is still reading. The epoch lives in device memory, so a captured CUDA graph replays it.
// A wait that gives up sets a status bit and the kernel still terminates.
#include "common.cuh"
#include "kernels.h"

namespace lb {

constexpr uint32_t TP_HEADER = 512;
constexpr uint32_t TP_SPIN_LIMIT = 1u << 21;

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256) tp_all_reduce_kernel(TpAllReduceArgs a) {
    __shared__ uint32_t s_epoch;
    __shared__ int s_ok;
    uint8_t *mine = (uint8_t *)a.peer[a.rank];
    uint32_t *flags = (uint32_t *)mine;
    uint32_t *epoch_ctr = (uint32_t *)(mine + 256), *done_ctr = epoch_ctr + 1;
    if (threadIdx.x == 0) {
        s_epoch = *(volatile uint32_t *)epoch_ctr + 1;  // every CTA reads it before the last one bumps it
        s_ok = 1;
    }
    __syncthreads();
    const uint32_t epoch = s_epoch, parity = epoch & 1;
    const uint32_t n4 = a.count / 4;
    const uint32_t per = (n4 + gridDim.x - 1) / gridDim.x;
    const uint32_t lo = blockIdx.x * per, hi = min(n4, lo + per);
    const size_t slot_floats = a.max_elems;

    // ---- push
    float4 *data4 = (float4 *)a.data;
    for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float4 v = data4[i];
        for (int q = 0; q < a.world; q++) {
            float4 *slot = (float4 *)((uint8_t *)a.peer[q] + TP_HEADER) + ((size_t)parity * a.world + a.rank) * (slot_floats / 4);
            slot[i] = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t prev = atomicAdd(done_ctr, 1u);
        if (prev == gridDim.x - 1) {
            *done_ctr = 0;
            *epoch_ctr = epoch;
            __threadfence_system();
            for (int q = 0; q < a.world; q++) st_release_sys((uint32_t *)a.peer[q] + a.rank, epoch);
        }
    }
    // ---- wait for every rank's push of this epoch
    if ((int)threadIdx.x < a.world) {
        bool ok = false;
        for (uint32_t spin = 0; spin < TP_SPIN_LIMIT; spin++) {
            if ((int32_t)(ld_acquire_sys(flags + threadIdx.x) - epoch) >= 0) {
                ok = true;
                break;
            }
            __nanosleep(40);
        }
        if (!ok) {
            s_ok = 0;
            if (a.status) atomicOr(a.status, 64);
        }
    }
    __syncthreads();
    // ---- reduce in rank order
    const float4 *base = (const float4 *)(mine + TP_HEADER) + (size_t)parity * a.world * (slot_floats / 4);
    for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        float4 acc = base[i];
        for (int q = 1; q < a.world; q++) {
            const float4 v = base[(size_t)q * (slot_floats / 4) + i];
            acc.x += v.x;
            acc.y += v.y;
            acc.z += v.z;
            acc.w += v.w;
        }
        data4[i] = acc;
    }
}

size_t tp_comm_bytes(int world, uint64_t max_elems) { return TP_HEADER + (size_t)2 * world * max_elems * 4; }

cudaError_t launch_tp_all_reduce(const TpAllReduceArgs &a, cudaStream_t stream) {
    if (a.count == 0) return cudaSuccess;
    if (a.count % 4 || a.count > a.max_elems || a.world < 1 || a.world > TP_MAX_RANKS) return cudaErrorInvalidValue;
    // few CTAs: the data is tens of KB at decode sizes; at prefill sizes use more to spread the peer stores
    uint32_t n4 = (uint32_t)(a.count / 4);
    uint32_t grid = (n4 + 1023) / 1024;
    if (grid < 1) grid = 1;
    if (grid > 64) grid = 64;  // all CTAs must be resident at once: the wait phase spins
    tp_all_reduce_kernel<<<grid, 256, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace lb

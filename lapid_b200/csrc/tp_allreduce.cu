// One-shot all-reduce (f32 sum, in place) of a row-parallel projection's partial results over the
// GPUs of one NVLink/NVSwitch domain, through peer-mapped memory. The reference has no multi-GPU
// code; this replaces a library all-reduce whose latency (tens of microseconds per call inside a
// token that needs two calls per layer) dominates tensor-parallel decode.
//
// Every rank owns one "symmetric" buffer, mapped into every peer's address space:
//     [0, 256)      TpPushTable: the peers' addresses, for kernels that hand over their result themselves
//     [256, 512)    epoch, done  u32: this rank's call counter and its CTA-completion counter
//     [512, ...)    slots[parity][src][max_elems]  of {f32 value, u32 epoch} pairs
// Every value travels with its own flag: a slot element is an 8-byte pair {value, epoch of the
// call}, and two neighbouring pairs go out as one 16-byte store. A receiver polls the pair itself
// until its flag shows the current epoch, so a call costs ONE one-way trip over NVLink: there is no
// separate "data complete" flag, hence no fence waiting for the remote writes to be acknowledged
// before a flag may follow them. (An 8-byte aligned store is never torn, so a pair whose flag has
// arrived carries its value; the two pairs of a 16-byte store are checked separately.)
// One kernel per call, no grid-wide barrier:
//   push    each thread stores its pairs of the local partial into slot[rank] of EVERY rank's
//           buffer (its own included): plain peer stores, 64 KB per peer at decode sizes
//   reduce  each thread polls the `world` slots of its own elements in its own buffer (bounded),
//           sums them in rank order and writes the result over the local partial: all ranks add
//           the same numbers in the same order, so the result is bit-identical everywhere
// Slots are double-buffered by epoch parity: a rank can be at most one call ahead of a peer (it
// cannot finish call e+1 before the peer has pushed its e+1 data, which the peer does only after it
// has finished reading call e), so it never overwrites a slot a peer is still reading. The epoch
// lives in device memory, so a captured CUDA graph replays it. The kernel opens with the
// programmatic-dependent-launch wait, so it may be queued behind the GEMV that produces the partial
// without a full drain. A poll that gives up sets a status bit and the kernel still terminates.
#include "common.cuh"
#include "kernels.h"
#include "tp_ll.cuh"

namespace lb {

// The same protocol has two more users: a decode GEMV can push its result straight from its
// epilogue (qgemv_q4k.cu, qgemv_q4k_mma.cu: GemvArgs::tp) and the normalisation that follows a
// row-parallel projection can poll and sum the slots itself (glue.cu: RmsNormArgs::tp), so that the
// all-reduce of a decode step costs no kernel of its own. `push_only` below is the fallback
// producer for launches whose kernel has no pushing epilogue.

__global__ void __launch_bounds__(256) tp_all_reduce_kernel(TpAllReduceArgs a) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ uint32_t s_epoch;
    uint8_t *mine = (uint8_t *)a.peer[a.rank];
    uint32_t *epoch_ctr = (uint32_t *)(mine + 256), *done_ctr = epoch_ctr + 1;
    if (threadIdx.x == 0) s_epoch = *(volatile uint32_t *)epoch_ctr + 1;  // every CTA reads it before the last one bumps it
    __syncthreads();
    const uint32_t epoch = s_epoch, parity = epoch & 1;
    const uint32_t n2 = (uint32_t)(a.count / 2);  // pairs of values = 16-byte slot stores
    const size_t slot_bytes = (size_t)a.max_elems * 8;
    const uint32_t stride = gridDim.x * blockDim.x, first = blockIdx.x * blockDim.x + threadIdx.x;

    // ---- push
    const float2 *data2 = (const float2 *)a.data;
    for (uint32_t i = first; i < n2; i += stride) {
        const float2 v = data2[i];
        for (int q = 0; q < a.world; q++)
            st_pairs((uint8_t *)a.peer[q] + TP_HEADER + ((size_t)parity * a.world + a.rank) * slot_bytes + (size_t)i * 16, v.x, v.y, epoch);
    }
    if (a.push_only) return;  // the reader closes the call (bumps the epoch)
    // ---- poll and reduce in rank order
    bool ok = true;
    const uint32_t limit = a.spin_limit ? a.spin_limit : TP_SPIN_LIMIT;
    const uint8_t *base = mine + TP_HEADER + (size_t)parity * a.world * slot_bytes;
    for (uint32_t i = first; i < n2; i += stride) {
        float2 acc = make_float2(0.0f, 0.0f);
        for (int q = 0; q < a.world; q++) {
            const uint8_t *src = base + (size_t)q * slot_bytes + (size_t)i * 16;
            uint4 v = ld_pairs(src);
            for (uint32_t spin = 0; ok && (v.y != epoch || v.w != epoch); spin++) {
                if (spin >= limit) {
                    ok = false;
                    break;
                }
                __nanosleep(20);
                v = ld_pairs(src);
            }
            const float x = __uint_as_float(v.x), y = __uint_as_float(v.z);
            acc.x = q ? acc.x + x : x;
            acc.y = q ? acc.y + y : y;
        }
        ((float2 *)a.data)[i] = acc;
    }
    if (!ok && a.status) atomicOr(a.status, 64);
    // ---- the last CTA to finish records the call
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t prev = atomicAdd(done_ctr, 1u);
        if (prev == gridDim.x - 1) {
            *done_ctr = 0;
            *(volatile uint32_t *)epoch_ctr = epoch;
        }
    }
}

size_t tp_comm_bytes(int world, uint64_t max_elems) { return TP_HEADER + (size_t)2 * world * max_elems * 8; }

cudaError_t launch_tp_all_reduce(const TpAllReduceArgs &a, bool pdl, cudaStream_t stream) {
    if (a.count == 0) return cudaSuccess;
    if (a.count % 4 || a.count > a.max_elems || a.world < 1 || a.world > TP_MAX_RANKS) return cudaErrorInvalidValue;
    // one pair of values per thread at decode sizes; every CTA must be resident at once (the
    // reduce phase polls), so the grid stays far below one CTA per SM slot
    const uint32_t n2 = (uint32_t)(a.count / 2);
    uint32_t grid = (n2 + 255) / 256;
    if (grid > 128) grid = 128;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, tp_all_reduce_kernel, a);
}

}  // namespace lb

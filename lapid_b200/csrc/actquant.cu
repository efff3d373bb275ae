// Activation rows -> int8 per 32-element group, the pre-pass of the decode path.
//
// Arithmetic of lapid-cpu's `quantize_row_scalar` (crates/lapid-cpu/src/matmul/quant.rs:68-89):
//   amax = max |x| over the group (NaN ignored), d = amax / 127, id = d > 0 ? 1/d : 0,
//   q = clamp(i32((x*id + 12582912.0) - 12582912.0), -127, 127)   (round half to even),
//   s[g] = d (f32), bs[g] = d * f32(sum q)   (bs only for weight formats with a min term).
// Note x * (1/(amax/127)), not x * (127/amax): the two differ in the last bit.
//
// One warp per group: lane t owns element t; max and sum are warp reductions (both are
// order-independent: max of floats, sum of small integers). The kernel moves 5.25 bytes per
// element and is latency-bound at decode sizes; what matters is that it is a single short wave.
#include "common.cuh"
#include "kernels.h"

namespace lb {

// One 32-element group of one row, by one warp.
__device__ __forceinline__ void quantize_group(const ActQuantArgs &p, uint32_t r, uint32_t g, int lane) {
    const uint32_t kg = p.k / GROUP;
    const void *row = act_row(p.a, p.a_type, p.a_off, p.a_bs, p.a_rs, r, p.m);
    float x = load_act(row, g * GROUP + lane, p.a_type);
    float amax = fabsf(x);
    if (!(amax == amax)) amax = 0.0f;  // f32::max ignores a NaN operand
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float d = xdiv(amax, 127.0f);
    float id = d > 0.0f ? xdiv(1.0f, d) : 0.0f;
    float rr = xsub(xadd(xmul(x, id), 12582912.0f), 12582912.0f);
    int q = (rr != rr) ? 0 : (int)rr;  // `as i32`: NaN -> 0, saturating
    q = q < -127 ? -127 : (q > 127 ? 127 : q);
    int sum = q;
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (p.records == 2) {
        // tiles of the tensor-core decode kernels: per super-block [sub-block][row][32] quants, then the group scales as
        // [sub-block pair 4][row pair 4][sub-block & 1][row & 1] (the four row pairs of a sub-block pair are 64
        // consecutive bytes: the lanes' 128-bit reads of them hit distinct banks) and the same for d * sum(q)
        const uint32_t sb = g & 7;
        uint8_t *blk = (uint8_t *)p.qa + (uint64_t)(g >> 3) * (256 * p.rows + 512);
        blk[(sb * p.rows + r) * 32 + lane] = (uint8_t)(int8_t)q;
        if (lane == 0) {
            float *sc = (float *)(blk + 256 * p.rows) + (((sb >> 1) * 4 + (r >> 1)) * 2 + (sb & 1)) * 2 + (r & 1);
            sc[0] = d;
            sc[64] = xmul(d, (float)sum);
        }
    } else if (p.records) {
        uint8_t *rec = (uint8_t *)p.qa + ((uint64_t)r * (p.k / QK) + (g >> 3)) * REC + 80 * ((g & 7) >> 1);
        rec[32 * (g & 1) + lane] = (uint8_t)(int8_t)q;
        if (lane == 0) {
            *(float *)(rec + 64 + 4 * (g & 1)) = d;
            *(float *)(rec + 72 + 4 * (g & 1)) = xmul(d, (float)sum);
        }
    } else {
        p.qa[(uint64_t)r * p.k + g * GROUP + lane] = (int8_t)q;
        if (lane == 0) {
            p.da[(uint64_t)r * kg + g] = d;
            if (p.bs) p.bs[(uint64_t)r * kg + g] = xmul(d, (float)sum);
        }
    }
}

__global__ void __launch_bounds__(256) act_quant_kernel(ActQuantArgs p) {
    // Under programmatic dependent launch: let the consumer's CTAs start staging weights now,
    // and do not read the activations before the producer grid has completed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const uint32_t kg = p.k / GROUP;
    const uint64_t n_groups = (uint64_t)p.rows * kg;
    const uint64_t warps = (uint64_t)gridDim.x * (blockDim.x >> 5);
    for (uint64_t gi = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); gi < n_groups; gi += warps)
        quantize_group(p, (uint32_t)(gi / kg), (uint32_t)(gi % kg), lane);
}

// Several independent activation operands in one launch (the pre-passes of a launch list whose
// inputs are not produced inside the list).
__global__ void __launch_bounds__(256) act_quant_batch_kernel(ActQuantBatch b) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const uint64_t total = b.group_end[b.count - 1];
    const uint64_t warps = (uint64_t)gridDim.x * (blockDim.x >> 5);
    for (uint64_t gi = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); gi < total; gi += warps) {
        int e = 0;
        while (gi >= b.group_end[e]) e++;
        const uint64_t local = gi - (e ? b.group_end[e - 1] : 0);
        const uint32_t kg = b.item[e].k / GROUP;
        quantize_group(b.item[e], (uint32_t)(local / kg), (uint32_t)(local % kg), lane);
    }
}

static cudaError_t launch_cfg(uint64_t n_groups, int sm_count, bool pdl, cudaStream_t stream, cudaLaunchConfig_t &cfg,
                              cudaLaunchAttribute *attr) {
    uint64_t ctas = (n_groups + 7) / 8;
    uint64_t cap = (uint64_t)sm_count * 8;
    cfg = {};
    cfg.gridDim = dim3((unsigned)(ctas < cap ? ctas : cap));
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaSuccess;
}

cudaError_t launch_act_quant(const ActQuantArgs &args, int sm_count, bool pdl, cudaStream_t stream) {
    uint64_t n_groups = (uint64_t)args.rows * (args.k / GROUP);
    if (n_groups == 0) return cudaSuccess;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    launch_cfg(n_groups, sm_count, pdl, stream, cfg, attr);
    return cudaLaunchKernelEx(&cfg, act_quant_kernel, args);
}

cudaError_t launch_act_quant_batch(const ActQuantBatch &batch, int sm_count, bool pdl, cudaStream_t stream) {
    if (batch.count <= 0 || batch.group_end[batch.count - 1] == 0) return cudaSuccess;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    launch_cfg(batch.group_end[batch.count - 1], sm_count, pdl, stream, cfg, attr);
    return cudaLaunchKernelEx(&cfg, act_quant_batch_kernel, batch);
}

}  // namespace lb

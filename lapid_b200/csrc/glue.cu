// The two row/elementwise steps that sit between the projections of a decoder layer, so that a
// layer-stack measurement is not dominated by a framework's many small kernels:
//
//   rms_norm   h = x (+ residual);  out = h * rsqrt(mean(h^2) + eps) (* weight)      per row
//              lapid's Kernel::RmsNorm (crates/lapid-compiler/src/ir.rs:407-409; CPU:
//              crates/lapid-cpu/src/rows.rs:118-156: f32 sum of squares, 1/sqrt, x * rstd * w),
//              with the residual add that precedes it in a layer folded in (optionally also
//              storing h, the new residual stream)
//   silu_mul   out = silu(gate) * up = gate / (1 + exp(-gate)) * up                   elementwise
//              the SwiGLU product (crates/lapid-nn/src/mlp.rs:84), an Elementwise kernel in lapid
//
// Both are memory-trivial (tens of KB at decode sizes) and latency-bound: one block per row with
// 128-bit accesses and a single block reduction, programmatic dependent launch like the GEMVs.
// They are not part of the quantized-matmul path; f32 results, not bit-matched to lapid-cpu (the
// order of the sum of squares differs): the tests hold them to 1e-5 relative against f64.
#include "common.cuh"
#include "kernels.h"

namespace lb {

constexpr int GLUE_THREADS = 256;
constexpr int GLUE_MAX_VEC = 16;  // float4 per thread kept in registers: cols <= 256 * 16 * 4 = 16384

__global__ void __launch_bounds__(GLUE_THREADS) rms_norm_kernel(RmsNormArgs p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float partial[GLUE_THREADS / 32];
    const uint32_t row = blockIdx.x, n4 = p.cols / 4;
    const float4 *x = (const float4 *)(p.x + (size_t)row * p.cols);
    const float4 *res = p.residual ? (const float4 *)(p.residual + (size_t)row * p.cols) : nullptr;
    float4 v[GLUE_MAX_VEC];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < GLUE_MAX_VEC; i++) {
        const uint32_t c = threadIdx.x + i * GLUE_THREADS;
        if (c < n4) {
            float4 a = x[c];
            if (res) {
                const float4 b = res[c];
                a.x += b.x;
                a.y += b.y;
                a.z += b.z;
                a.w += b.w;
            }
            if (p.sum_out) ((float4 *)(p.sum_out + (size_t)row * p.cols))[c] = a;
            v[i] = a;
            ss = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, fmaf(a.w, a.w, ss))));
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < GLUE_THREADS / 32; w++) tot += partial[w];
    const float rstd = 1.0f / sqrtf(tot * (1.0f / (float)p.cols) + p.eps);
#pragma unroll
    for (int i = 0; i < GLUE_MAX_VEC; i++) {
        const uint32_t c = threadIdx.x + i * GLUE_THREADS;
        if (c < n4) {
            float4 a = v[i];
            a.x *= rstd;
            a.y *= rstd;
            a.z *= rstd;
            a.w *= rstd;
            if (p.weight) {
                const float4 g = ((const float4 *)p.weight)[c];
                a.x *= g.x;
                a.y *= g.y;
                a.z *= g.z;
                a.w *= g.w;
            }
            ((float4 *)(p.out + (size_t)row * p.cols))[c] = a;
        }
    }
}

__global__ void __launch_bounds__(GLUE_THREADS) silu_mul_kernel(const float *gate, const float *up, float *out, uint64_t n4) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint64_t i = (uint64_t)blockIdx.x * GLUE_THREADS + threadIdx.x; i < n4; i += (uint64_t)gridDim.x * GLUE_THREADS) {
        const float4 g = ((const float4 *)gate)[i], u = ((const float4 *)up)[i];
        float4 o;
        o.x = g.x / (1.0f + expf(-g.x)) * u.x;
        o.y = g.y / (1.0f + expf(-g.y)) * u.y;
        o.z = g.z / (1.0f + expf(-g.z)) * u.z;
        o.w = g.w / (1.0f + expf(-g.w)) * u.w;
        ((float4 *)out)[i] = o;
    }
}

static void pdl_config(cudaLaunchConfig_t &cfg, cudaLaunchAttribute *attr, unsigned grid, bool pdl, cudaStream_t stream) {
    cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(GLUE_THREADS);
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
}

bool rms_norm_shape_ok(uint32_t cols) { return cols >= 4 && cols % 4 == 0 && cols <= GLUE_THREADS * GLUE_MAX_VEC * 4; }

cudaError_t launch_rms_norm(const RmsNormArgs &a, bool pdl, cudaStream_t stream) {
    if (a.rows == 0) return cudaSuccess;
    if (!rms_norm_shape_ok(a.cols)) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    pdl_config(cfg, attr, a.rows, pdl, stream);
    return cudaLaunchKernelEx(&cfg, rms_norm_kernel, a);
}

cudaError_t launch_silu_mul(const float *gate, const float *up, float *out, uint64_t n, int sm_count, bool pdl, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    if (n % 4) return cudaErrorInvalidValue;
    const uint64_t n4 = n / 4, want = (n4 + GLUE_THREADS - 1) / GLUE_THREADS, cap = (uint64_t)sm_count * 8;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    pdl_config(cfg, attr, (unsigned)(want < cap ? want : cap), pdl, stream);
    return cudaLaunchKernelEx(&cfg, silu_mul_kernel, gate, up, out, n4);
}

}  // namespace lb

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
// Both are memory-trivial (tens of KB at decode sizes) and latency-bound: 128-bit accesses, a row
// is split over a thread-block cluster of up to 8 CTAs whose partial sums of squares meet through
// distributed shared memory (so a single decode row still spreads over 8 SMs -- which matters most
// when the row is the sum of the tensor-parallel ranks' partials, polled from the hand-off slots),
// programmatic dependent launch like the GEMVs.
// They are not part of the quantized-matmul path; f32 results, not bit-matched to lapid-cpu (the
// order of the sum of squares differs): the tests hold them to 1e-5 relative against f64.
#include <cooperative_groups.h>

#include "actquant.cuh"
#include "common.cuh"
#include "kernels.h"
#include "tp_ll.cuh"

namespace cg = cooperative_groups;

namespace lb {

constexpr int GLUE_THREADS = 256;
constexpr int GLUE_MAX_VEC = 16;  // float4 per thread kept in registers: cols <= 256 * 16 * 4 = 16384

__global__ void __launch_bounds__(GLUE_THREADS) rms_norm_kernel(RmsNormArgs p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float partial[GLUE_THREADS / 32];
    __shared__ float cta_ss;
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t parts = cluster.num_blocks(), part = cluster.block_rank();
    const uint32_t row = blockIdx.x / parts, n4 = p.cols / 4;
    const uint32_t per = (n4 + parts - 1) / parts, c_lo = part * per, c_hi = min(n4, c_lo + per);  // this CTA's float4 columns
    // tensor-parallel input: x = sum over ranks (in rank order) of the partials they pushed for the
    // call in progress, polled pair by pair from this rank's own slots (protocol: tp_allreduce.cu)
    uint32_t epoch = 0;
    const uint8_t *slots = nullptr;
    size_t slot_bytes = 0;
    bool ok = true;
    if (p.tp) {
        epoch = tp_current_epoch(p.tp);
        slot_bytes = (size_t)p.tp->max_elems * 8;
        slots = (const uint8_t *)p.tp->peer[p.tp->rank] + TP_HEADER + (size_t)(epoch & 1) * p.tp->world * slot_bytes +
                (size_t)row * p.cols * 8;
    }
    const float4 *x = (const float4 *)(p.x + (size_t)row * p.cols);
    const float4 *res = p.residual ? (const float4 *)(p.residual + (size_t)row * p.cols) : nullptr;
    float4 v[GLUE_MAX_VEC];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < GLUE_MAX_VEC; i++) {
        const uint32_t c = c_lo + threadIdx.x + i * GLUE_THREADS;
        if (c < c_hi) {
            float4 a;
            if (p.tp) {
                a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int q = 0; q < p.tp->world; q++) {
                    const uint8_t *src = slots + (size_t)q * slot_bytes + (size_t)c * 32;
                    uint4 lo = ld_pairs(src), hi = ld_pairs(src + 16);
                    for (uint32_t spin = 0; ok && (lo.y != epoch || lo.w != epoch || hi.y != epoch || hi.w != epoch); spin++) {
                        if (spin >= (p.spin_limit ? p.spin_limit : TP_SPIN_LIMIT)) {
                            ok = false;
                            break;
                        }
                        __nanosleep(20);
                        lo = ld_pairs(src);
                        hi = ld_pairs(src + 16);
                    }
                    const float4 v = make_float4(__uint_as_float(lo.x), __uint_as_float(lo.z), __uint_as_float(hi.x), __uint_as_float(hi.z));
                    a.x = q ? a.x + v.x : v.x;
                    a.y = q ? a.y + v.y : v.y;
                    a.z = q ? a.z + v.z : v.z;
                    a.w = q ? a.w + v.w : v.w;
                }
            } else {
                a = x[c];
            }
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
    if (parts > 1) {  // every CTA of the row adds the partial sums in the same order
        if (threadIdx.x == 0) cta_ss = tot;
        cluster.sync();
        tot = 0.0f;
        for (uint32_t r = 0; r < parts; r++) tot += *cluster.map_shared_rank(&cta_ss, r);
    }
    const float rstd = 1.0f / sqrtf(tot * (1.0f / (float)p.cols) + p.eps);
#pragma unroll
    for (int i = 0; i < GLUE_MAX_VEC; i++) {
        const uint32_t c = c_lo + threadIdx.x + i * GLUE_THREADS;
        const bool active = c < c_hi;
        float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (active) {
            a = v[i];
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
        // the same values as the int8 operand of the GEMVs that read `out` (warp-uniform branch: whole warps of
        // the CTA's column range take it together, lanes past the range pass active = false)
        if (p.q.qa && c_lo + (threadIdx.x & ~31u) + i * GLUE_THREADS < c_hi) act_quant_quad(p.q, active, row, 4 * c, a);
    }
    if (parts > 1) cluster.sync();  // no CTA leaves while a neighbour may still read its partial sum
    if (p.tp) {  // the last CTA to finish closes the call
        if (!ok && p.status) atomicOr(p.status, 64);
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t *epoch_ctr = (uint32_t *)((uint8_t *)p.tp->peer[p.tp->rank] + 256), *done_ctr = epoch_ctr + 1;
            if (atomicAdd(done_ctr, 1u) == gridDim.x - 1) {
                *done_ctr = 0;
                *(volatile uint32_t *)epoch_ctr = epoch;
            }
        }
    }
}

__global__ void __launch_bounds__(GLUE_THREADS) silu_mul_kernel(const float *gate, const float *up, float *out, uint64_t n4, uint32_t cols4,
                                                                ActOut q) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // whole warps iterate together (the quantized copy needs every lane of a warp in the call)
    for (uint64_t base = (uint64_t)blockIdx.x * GLUE_THREADS + (threadIdx.x & ~31u); base < n4; base += (uint64_t)gridDim.x * GLUE_THREADS) {
        const uint64_t i = base + (threadIdx.x & 31u);
        const bool active = i < n4;
        float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (active) {
            const float4 g = ((const float4 *)gate)[i], u = ((const float4 *)up)[i];
            o.x = g.x / (1.0f + expf(-g.x)) * u.x;
            o.y = g.y / (1.0f + expf(-g.y)) * u.y;
            o.z = g.z / (1.0f + expf(-g.z)) * u.z;
            o.w = g.w / (1.0f + expf(-g.w)) * u.w;
            ((float4 *)out)[i] = o;
        }
        if (q.qa) act_quant_quad(q, active, (uint32_t)(i / cols4), 4 * (uint32_t)(i % cols4), o);
    }
}

static void pdl_config(cudaLaunchConfig_t &cfg, cudaLaunchAttribute *attr, unsigned grid, bool pdl, cudaStream_t stream,
                       unsigned cluster = 1) {
    cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(GLUE_THREADS);
    cfg.stream = stream;
    int n = 0;
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    if (cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        n++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
}

bool rms_norm_shape_ok(uint32_t cols) { return cols >= 4 && cols % 4 == 0 && cols <= GLUE_THREADS * GLUE_MAX_VEC * 4; }

static unsigned rms_norm_parts(uint32_t cols) { return cols >= 4096 ? 8 : cols >= 2048 ? 4 : cols >= 1024 ? 2 : 1; }

// every CTA of the cluster gets whole 32-element groups, in whole blocks of the quantized layouts
bool rms_norm_quant_ok(uint32_t cols) { return rms_norm_shape_ok(cols) && cols % QK == 0 && (cols / 4) % (8 * rms_norm_parts(cols)) == 0; }

cudaError_t launch_rms_norm(const RmsNormArgs &a, bool pdl, cudaStream_t stream) {
    if (a.rows == 0) return cudaSuccess;
    if (!rms_norm_shape_ok(a.cols)) return cudaErrorInvalidValue;
    if (a.q.qa && (!rms_norm_quant_ok(a.cols) || a.q.k != a.cols || a.q.rows != a.rows)) return cudaErrorInvalidValue;
    const unsigned parts = rms_norm_parts(a.cols);
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    pdl_config(cfg, attr, a.rows * parts, pdl, stream, parts);
    return cudaLaunchKernelEx(&cfg, rms_norm_kernel, a);
}

cudaError_t launch_silu_mul(const float *gate, const float *up, float *out, uint64_t n, uint32_t cols, const ActOut &q, int sm_count,
                            bool pdl, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    if (n % 4) return cudaErrorInvalidValue;
    if (q.qa && (cols == 0 || cols % QK != 0 || n % cols != 0 || q.k != cols || (uint64_t)q.rows * cols != n)) return cudaErrorInvalidValue;
    const uint64_t n4 = n / 4, want = (n4 + GLUE_THREADS - 1) / GLUE_THREADS, cap = (uint64_t)sm_count * 8;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    pdl_config(cfg, attr, (unsigned)(want < cap ? want : cap), pdl, stream);
    return cudaLaunchKernelEx(&cfg, silu_mul_kernel, gate, up, out, n4, q.qa ? cols / 4 : 1u, q);
}

// ---- the epilogue expression of a prefill launch, applied to its output in place (the GEMM kernels store the plain
//      accumulators first; the decode kernels evaluate the expression in their own stores)
__global__ void __launch_bounds__(256) epilogue_expr_kernel(EpiProg prog, float *out, uint64_t out_off, uint64_t out_bs, uint64_t out_rs,
                                                            const float *extra, uint64_t ex_off, int64_t ex_s0, int64_t ex_s1, int64_t ex_s2,
                                                            uint32_t batch, uint32_t m, uint32_t n) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint64_t total = (uint64_t)batch * m * n;
    for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = e / n, j = e - row * n, bt = row / m, i = row - bt * m;
        float *o = out + out_off + bt * out_bs + i * out_rs + j;
        const float x = extra ? extra[(int64_t)ex_off + (int64_t)bt * ex_s0 + (int64_t)i * ex_s1 + (int64_t)j * ex_s2] : 0.0f;
        *o = epi_eval(prog, *o, x);
    }
}

cudaError_t launch_epilogue_expr(const EpiProg &prog, float *out, uint64_t out_off, uint64_t out_bs, uint64_t out_rs, const float *extra,
                                 uint64_t ex_off, int64_t ex_s0, int64_t ex_s1, int64_t ex_s2, uint32_t batch, uint32_t m, uint32_t n,
                                 int sm_count, cudaStream_t stream) {
    const uint64_t total = (uint64_t)batch * m * n;
    if (!total || !prog.n) return cudaSuccess;
    uint64_t blocks = (total + 255) / 256;
    if (blocks > (uint64_t)sm_count * 16) blocks = (uint64_t)sm_count * 16;
    epilogue_expr_kernel<<<(unsigned)blocks, 256, 0, stream>>>(prog, out, out_off, out_bs, out_rs, extra, ex_off, ex_s0, ex_s1, ex_s2, batch, m, n);
    return cudaGetLastError();
}

}  // namespace lb

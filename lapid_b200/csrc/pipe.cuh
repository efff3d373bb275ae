// Device helpers of the shared-memory pipelines: mbarriers with bounded waits, the bulk-copy and
// tensor-map (TMA) loads that complete on them, the warp-level int8 tensor-core instruction and
// Blackwell's packed f32x2 arithmetic.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lb {
namespace pipe {

__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(bar)) : "memory");
}
// Bounded wait for the phase with the given parity; false when it gave up after `limit` polls.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = 1u << 22) {
    for (uint32_t spin = 0; spin < limit; spin++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(s32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
// Contiguous global -> shared copy by the bulk-copy engine: both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(s32(dst)),
                 "l"(src), "r"(bytes), "r"(s32(bar))
                 : "memory");
}
// One box of a 2-D tensor map; x (innermost coordinate) times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     s32(dst)),
                 "l"((uint64_t)map), "r"(x), "r"(y), "r"(s32(bar))
                 : "memory");
}

// 16 weight rows (unsigned bytes) x 32 k x 8 activation rows (signed bytes). The accumulators start at
// the bit pattern of 1.5 * 2^23: the integer dot product (|dot| < 2^22) lands in the mantissa, so the
// result reinterpreted as f32 is 12582912 + dot and one exact addition replaces the int -> float step.
constexpr float MAGIC = 12582912.0f;
__device__ __forceinline__ void mma_u8s8_magic(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0x4B400000));
}

// Two f32 lanes in one 64-bit register pair.
__device__ __forceinline__ uint64_t pack2i(int lo, int hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// float(byte `sel` of w) * d, exactly: the byte is planted in the mantissa of 2^23 with one PRMT and the
// bias is removed inside one fused multiply-add (d * (2^23 + b) - d * 2^23 = d * b needs 17 bits).
__device__ __forceinline__ float scale_byte(uint32_t w, uint32_t sel, float d, float neg_d23) {
    return fmaf(d, __uint_as_float(__byte_perm(w, 0x4B000000u, sel)), neg_d23);
}

}  // namespace pipe
}  // namespace lb

// Device helpers of the tensor-parallel hand-off (protocol: tp_allreduce.cu). A slot element is an
// 8-byte pair {f32 value, u32 epoch of the call}; a pair whose flag shows the current epoch carries
// its value (an aligned 8-byte store is never torn).
#pragma once
#include <cstdint>

#include "kernels.h"

namespace lb {

constexpr uint32_t TP_HEADER = 512;      // [0, 256) TpPushTable, [256, 512) epoch and done counters, then the slots
constexpr uint32_t TP_SPIN_LIMIT = 1u << 21;

__device__ __forceinline__ void st_pair(void *p, float a, uint32_t epoch) {
    asm volatile("st.volatile.global.v2.b32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(a)), "r"(epoch) : "memory");
}
__device__ __forceinline__ void st_pairs(void *p, float a, float b, uint32_t epoch) {
    asm volatile("st.volatile.global.v4.b32 [%0], {%1, %2, %3, %2};" ::"l"(p), "r"(__float_as_uint(a)), "r"(epoch), "r"(__float_as_uint(b))
                 : "memory");
}
__device__ __forceinline__ uint4 ld_pairs(const void *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// The epoch of the call in progress: one more than the last closed one. Read it only after the
// programmatic-dependent-launch wait (the kernel that closed the previous call must be complete).
__device__ __forceinline__ uint32_t tp_current_epoch(const TpPushTable *tp) {
    return *(volatile const uint32_t *)((const uint8_t *)tp->peer[tp->rank] + 256) + 1;
}
// What a pushing kernel keeps in shared memory: read once per CTA (after the dependent-launch wait),
// so that an epilogue store costs no dependent global loads.
struct TpPushCtx {
    uint8_t *slot[TP_MAX_RANKS];  // this rank's slot of the call in progress, in every rank's buffer
    uint32_t epoch;
    int32_t world;
};
__device__ __forceinline__ void tp_push_ctx_load(TpPushCtx *ctx, const TpPushTable *tp) {
    const uint32_t epoch = tp_current_epoch(tp);
    const size_t off = TP_HEADER + ((size_t)(epoch & 1) * tp->world + tp->rank) * (tp->max_elems * 8);
    for (int q = 0; q < tp->world; q++) ctx->slot[q] = (uint8_t *)tp->peer[q] + off;
    ctx->epoch = epoch;
    ctx->world = tp->world;
}
// One value of this rank's result, element `idx` of the row-major result, to every rank.
__device__ __forceinline__ void tp_push_value(const TpPushCtx *ctx, uint64_t idx, float v) {
    for (int q = 0; q < ctx->world; q++) st_pair(ctx->slot[q] + idx * 8, v, ctx->epoch);
}

}  // namespace lb

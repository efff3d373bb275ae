// Host-callable launchers of the CUDA kernels. Everything here is asynchronous on `stream`.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

namespace lb {

// A fused epilogue expression (MatMulSpec.epilogue, crates/lapid-compiler/src/ir.rs:94-111 restricted to its f32 part) as
// a postfix program over Load(0) = the accumulator and Load(1) = extras[0]: `code[i]` = op | arg << 8; EPI_CONST is
// followed by the constant's bits. n == 0: no program (the launch's `extra`, if any, is added). Evaluated with a
// four-deep register stack (epi_eval in common.cuh); the host checks the stack discipline before a launch.
constexpr int EPI_WORDS = 24;
enum : uint32_t {
    EPI_LOAD = 1, EPI_CONST = 2,
    EPI_NEG = 16, EPI_EXP, EPI_LOG, EPI_SQRT, EPI_RSQRT, EPI_RECIP, EPI_SIN, EPI_COS, EPI_TANH, EPI_ERF, EPI_ABS, EPI_UNARY_END,
    EPI_ADD = 32, EPI_SUB, EPI_MUL, EPI_DIV, EPI_MAX, EPI_MIN, EPI_POW, EPI_CMPLT, EPI_CMPEQ, EPI_BINARY_END,
    EPI_WHERE = 48,
};
struct EpiProg {
    uint32_t n;
    uint32_t code[EPI_WORDS];
};
// Applies `prog` to out[bt, i, j] in place (the prefill kernels run their GEMM first): rows x n elements.
cudaError_t launch_epilogue_expr(const EpiProg &prog, float *out, uint64_t out_off, uint64_t out_bs, uint64_t out_rs, const float *extra,
                                 uint64_t ex_off, int64_t ex_s0, int64_t ex_s1, int64_t ex_s2, uint32_t batch, uint32_t m, uint32_t n,
                                 int sm_count, cudaStream_t stream);

// ---- dequant.cu
cudaError_t launch_gather(int fmt, const void *table, uint64_t scales_offset, const int32_t *ids, uint64_t rows, uint64_t cols,
                          uint64_t count, float *out, int *status, int sm_count, cudaStream_t stream);  // fmt < 0: f32 table
cudaError_t launch_dequantize(int fmt, const void *src, uint64_t rows, uint64_t cols, uint64_t scales_offset,
                              float *dst, int sm_count, cudaStream_t stream);
cudaError_t launch_q8_0_to_planes(const void *blocks, void *dst, uint64_t scales_offset, uint64_t n_groups,
                                  int sm_count, cudaStream_t stream);
cudaError_t launch_q4_0_to_planes(const void *blocks, void *dst, uint64_t scales_offset, uint64_t n_groups,
                                  int sm_count, cudaStream_t stream);


// ---- quantize.cu
cudaError_t launch_quantize(int fmt, const float *src, uint64_t rows, uint64_t cols, uint64_t scales_offset,
                            uint64_t total_bytes, void *dst, int sm_count, cudaStream_t stream);

// ---- actquant.cu
// Activation rows -> int8 per 32-group. Row r = bt*m + i starts at a + a_off + bt*a_bs + i*a_rs.
// qa: [rows][k] int8; da: [rows][k/32] f32 group scales; bs: [rows][k/32] f32 = da * sum(q)
// (written only when bs != nullptr, i.e. for Q4_K weights).
struct ActQuantArgs {
    const void *a;          // f32, f16 or bf16 rows (a_type: ACT_F32 / ACT_F16 / ACT_BF16 of common.cuh), strides in elements
    int a_type;
    uint64_t a_off, a_bs, a_rs;
    uint32_t rows, m, k;
    int8_t *qa;
    float *da;
    float *bs;
    // records != 0: instead of the three planes, write one ACT_RECORD-byte record per
    // (row, 256-element block) at qa: four times [64 quants | da_2p da_2p+1 bs_2p bs_2p+1], 16 pad.
    int records;
};
constexpr int REC = 336;
// Where a producing kernel (glue.cu) leaves its result as the quantized operand of the decode GEMV that
// follows: the same layouts as ActQuantArgs (records 0: planes qa / da / bs; 1: records; 2: tiles, both at qa).
struct ActOut {
    int8_t *qa;  // nullptr: no quantized copy
    float *da;
    float *bs;
    int records;
    uint32_t rows, k;
};
// Bytes of a quantized activation operand and where its planes start (records == 0).
inline size_t act_plane_bytes(uint32_t rows, uint32_t k) { return (((size_t)rows * k + 255) & ~(size_t)255); }
inline size_t act_scale_bytes(uint32_t rows, uint32_t k) { return (((size_t)rows * (k / 32) * 4 + 255) & ~(size_t)255); }
cudaError_t launch_act_quant(const ActQuantArgs &args, int sm_count, bool pdl, cudaStream_t stream);
// Up to ACT_BATCH_MAX operands in one launch; group_end[i] = running total of 32-groups.
constexpr int ACT_BATCH_MAX = 24;
struct ActQuantBatch {
    ActQuantArgs item[ACT_BATCH_MAX];
    uint64_t group_end[ACT_BATCH_MAX];
    int count;
};
cudaError_t launch_act_quant_batch(const ActQuantBatch &batch, int sm_count, bool pdl, cudaStream_t stream);

// ---- qgemv.cu
// What a kernel needs to hand its result to the other ranks of a tensor-parallel group (see
// tp_allreduce.cu): lives in device memory, at the start of this rank's symmetric buffer.
constexpr int TP_MAX_RANKS = 8;
struct TpPushTable {
    void *peer[TP_MAX_RANKS];  // every rank's symmetric buffer as mapped on this GPU; peer[rank] is this rank's own
    uint64_t max_elems;        // value capacity of one slot
    int32_t rank, world;
};

struct GemvArgs {
    const uint8_t *w;       // quantized [n, k] matrix in lapid-quant layout
    uint64_t w_bytes;       // bytes readable behind `w`
    uint64_t scales_offset; // Int8 only
    const int8_t *qa;       // quantized activations, see ActQuantArgs
    const float *da;
    const float *bs;
    const float *a;         // f32 activations (kernels that quantize them in their prologue)
    uint64_t a_off, a_bs, a_rs;
    int *status;            // host-visible word; a kernel ORs a bit in when one of its bounded waits gave up
    float *out;             // row r = bt*m + i at out + out_off + bt*out_bs + i*out_rs
    uint64_t out_off, out_bs, out_rs;
    const float *extra;     // epilogue `acc + extra[bt, i, j]`, nullptr for none
    uint64_t ex_off;
    int64_t ex_s0, ex_s1, ex_s2;
    EpiProg epi;            // epi.n != 0: the epilogue is this expression over the accumulator and extra[bt, i, j] instead. A kernel
                            // then stores the plain accumulator (the host applies the expression with one more kernel) unless
                            // its launcher says it evaluates expressions itself (and clears epi.n in the caller's struct)
    uint32_t rows, m, n, k;
    const TpPushTable *tp;  // not nullptr (K-quant fast kernels only): the result, row-major [rows, n], goes to slot[rank] of every
                            // rank's buffer as {value, epoch} pairs instead of to `out`
    // Expert-indexed launches (launch_qgemv_kq_moe only): `w` is a stack of `id_e` matrices [n, k], `id_stride` bytes
    // apart; ids[t, id_r] (i32) picks the matrix of each (token, slot) pair; rows = tokens; out is [rows, id_r, n].
    const int32_t *ids;
    uint64_t id_stride;
    uint32_t id_r, id_e;
    uint32_t id_pairs;      // launch_qgemv_moe (generic kernel): tokens * id_r, one grid row each; `rows` is 1 there
    // 1: everything the kernel READS (weights, quantized activations) was complete before the kernel in front of it
    // in the stream started, so under programmatic dependent launch it may read and compute without waiting for that
    // kernel and only has to wait before it WRITES. Set by the host for launches whose activations were quantized by
    // the pre-pass at the head of an execute list, when a fully serialised launch lies in between. Kernels may ignore it.
    uint32_t early;
};
// rows in 1..8. Returns cudaErrorInvalidValue for an unsupported combination.
cudaError_t launch_qgemv(int fmt, const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream);
// Expert-indexed form of the same kernel for every format and K (args.ids set; args.rows = tokens, 1..8).
cudaError_t launch_qgemv_moe(int fmt, const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream);
// ---- qgemv_i4.cu: Int4 nibble planes, 1..8 rows (and the expert-indexed form: args.ids set, rows = tokens)
cudaError_t launch_qgemv_i4(const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream);
// ---- qgemv_mxfp4.cu: MXFP4 blocks, 1..8 rows (and the expert-indexed form: args.ids set, rows = tokens); reads the planes
cudaError_t launch_qgemv_mxfp4(const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream);
// qgemv_mxfp4_mma.cu: the same blocks on the int8 tensor-core instruction (K a multiple of 512; the activation tiles
// of the K-quant kernels)
bool qgemv_mxfp4_mma_shape_ok(uint32_t rows, uint32_t k);
cudaError_t launch_qgemv_mxfp4_mma(const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream);
void qgemv_mxfp4_set_k_split(int ways);  // warps per row of the direct form: 0: per launch (default); 1, 2, 4: forced
void qgemv_mxfp4_set_staged(int on);  // 1 (default): rows staged through shared memory where K allows; 0: direct loads only

// ---- qgemv_iq.cu: the grid-based i-quants (IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS), 1..8 rows (and the expert-indexed form);
// reads the activation planes, the codebooks from the per-device table of iquant.cu
cudaError_t launch_qgemv_iq(int fmt, const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream);
void qgemv_iq_set_rows_per_warp(int rows);  // 0: per launch (default); 1, 2: forced
void qgemv_iq_set_k_split(int ways);        // warps per row at one row per warp: 0: per launch (default); 1, 2, 4: forced
// iquant.cu: uploads the codebooks to the current device (once; outside stream captures)
cudaError_t iq_grids_upload();
// Opt in to the dynamic shared memory the GEMV variants need; once per device.
cudaError_t qgemv_init();

// ---- qgemv_q4k.cu: dp4a fast path for Q4_K and Q6_K, 1..8 rows (the default for one row)
// Reads the activations as 336-byte records (ActQuantArgs::records) from args.qa.
bool qgemv_q4k_fast_supported(const GemvArgs &args);
cudaError_t launch_qgemv_q4k_fast(const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream);
// The largest dynamic shared-memory size a kernel has been opted in to, per device of the process
// (cudaFuncSetAttribute is a per-device setting). Used as a function-local static by the launchers.
// Launches may come from several host threads (one per device): the table is guarded by its own mutex.
struct DynamicSmemOptIn {
    size_t have[64] = {};
    std::mutex mu;
    cudaError_t raise(const void *kernel, size_t bytes) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
        std::lock_guard<std::mutex> lock(mu);
        if (bytes <= have[dev]) return cudaSuccess;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e == cudaSuccess) have[dev] = bytes;
        return e;
    }
};

// Resident CTAs per SM of a kernel for a dynamic shared-memory size, remembered per (device, size); a launcher keeps
// one as a function-local static. Thread-safe; when the table is full the answer is computed every time.
struct OccupancyCache {
    struct Entry {
        int dev;
        size_t smem;
        int ctas;
    };
    Entry e[16];
    int n = 0;
    std::mutex mu;
    template <class K> cudaError_t get(K kernel, int threads, size_t smem, int *out) {
        int dev = 0;
        if (cudaError_t err = cudaGetDevice(&dev); err != cudaSuccess) return err;
        std::lock_guard<std::mutex> lock(mu);
        for (int i = 0; i < n; i++)
            if (e[i].dev == dev && e[i].smem == smem) {
                *out = e[i].ctas;
                return cudaSuccess;
            }
        int occ = 0;
        if (cudaError_t err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, threads, smem); err != cudaSuccess) return err;
        if (occ < 1) occ = 1;
        if (n < 16) e[n++] = Entry{dev, smem, occ};
        *out = occ;
        return cudaSuccess;
    }
};

// Up to GEMV_GROUP_MAX independent projections with the same format, rows and k in one launch.
constexpr int GEMV_GROUP_MAX = 6;
template <int N> struct GemvGroupT {
    GemvArgs item[N];
    uint32_t task_end[N];  // filled by the launcher
    uint32_t act_off[N];   // shared-memory offset of each item's activation records
    uint8_t act_copy[N];   // 0 when an earlier item of the group has the same activations
    int count;
    uint32_t act_bytes;
};
using GemvGroup = GemvGroupT<GEMV_GROUP_MAX>;
using GemvSingle = GemvGroupT<1>;  // what a lone launch passes to the kernel: a sixth of the parameter bytes
size_t qgemv_kq_group_smem(int fmt, GemvGroup &group);  // dynamic shared memory the group would need
cudaError_t launch_qgemv_kq_group(int fmt, GemvGroup &group, int sm_count, bool pdl, cudaStream_t stream);
// Q4_K decode on the warp-level int8 tensor-core instruction (2..8 rows pay off); activations as
// tiles (ActQuantArgs::records == 2).
bool qgemv_q4k_mma_shape_ok(uint32_t rows, uint32_t k);
size_t qgemv_q4k_mma_act_bytes(uint32_t rows, uint32_t k);
bool qgemv_q4k_mma_group_fits(GemvGroup &group);
struct StreamWs;
cudaError_t launch_qgemv_q4k_mma(GemvGroup &group, int sm_count, bool pdl, cudaStream_t stream, StreamWs *ws = nullptr);
void qgemv_q4k_mma_set_config(int index);  // -1 = pick by shared-memory fit
void qgemv_q6k_mma_set_config(int index);  // tuning: layout of the Q6_K tensor-core decode kernel, -1 = choose
// ---- qgemv_kq_stream.cu: Q4_K / Q5_K decode on the same instruction as one stream of equal work shares
// (2..8 rows; any K that is a multiple of 256; same activation tiles). One workspace per device serves every launch
// of its stream (all zero between launches): `pairs` ({f32 value, u32 flag}) through which the spans of a dependent
// launch hand partial tiles to each other, and behind it the staging regions of the launches that run ahead of their
// predecessor (control words + partial tiles), which the launcher hands out in rotation (launches of one device are
// serialised by its owner).
struct StreamWs {
    uint2 *pairs;
    uint64_t n_pairs;
    uint8_t *stage;        // STAGE_REGIONS x (control words, partial tiles)
    uint64_t total_bytes;  // of the whole allocation, from `pairs` on
    uint32_t next_region, next_id;
    uint64_t kernels;      // kernels launched through this workspace so far (a launch that runs ahead takes two)
};
// Diagnostics: per-CTA timeline rows of the next `launches` launches (16 words per CTA; see include/lapid_b200.h)
cudaError_t qgemv_kq_stream_trace_begin(uint32_t launches, int sm_count);
uint32_t qgemv_kq_stream_trace_read(unsigned long long *out, uint64_t cap_words, uint32_t *ctas);
size_t qgemv_kq_stream_ws_bytes(int sm_count, StreamWs *layout);  // bytes to allocate (zero-filled)
bool qgemv_kq_stream_shape_ok(int fmt, uint32_t rows, uint32_t n, uint32_t k);
cudaError_t launch_qgemv_kq_stream(int fmt, GemvGroup &group, StreamWs &ws, int sm_count, bool pdl, cudaStream_t stream);
void qgemv_kq_stream_set_config(int index);     // tuning: -1 = choose
void qgemv_kq_stream_set_ctas_per_sm(int n);    // tuning: 0 = choose
void qgemv_kq_stream_set_debug(int v);          // measurement only: 2 = drop partial tiles (wrong results)
void qgemv_kq_stream_set_final_tiles(int v);    // tuning: row tiles per finalising CTA of a launch that runs ahead (0 = choose)
void qgemv_kq_stream_set_spin_limit(int v);     // polls before the claim of a staging region gives up (0 = default)
void qgemv_kq_stream_set_big_units(int v);      // tuning: 128-row units per SM from which the 32-row warps are used
void qgemv_kq_stream_set_early_ctas(int v);     // tuning: CTAs per SM of a launch that runs ahead of its predecessor (0 = as any launch)
// Int4 nibble planes on the same instruction (qgemv_i4_mma.cu; K a multiple of 512); same activation tiles.
bool qgemv_i4_mma_shape_ok(uint32_t rows, uint32_t k);
cudaError_t launch_qgemv_i4_mma(const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream);
// Int8 planes on the same instruction (K a multiple of 512); same activation tiles.
bool qgemv_i8_mma_shape_ok(uint32_t rows, uint32_t k);
cudaError_t launch_qgemv_i8_mma(const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream);
// Its Q6_K sibling (K a multiple of 2048); same activation tiles.
bool qgemv_q6k_mma_shape_ok(uint32_t rows, uint32_t k);
bool qgemv_q6k_mma_group_fits(GemvGroup &group);
cudaError_t launch_qgemv_q6k_mma(GemvGroup &group, int sm_count, bool pdl, cudaStream_t stream);
bool qgemv_kq_fast_supported(int fmt, const GemvArgs &args);  // Q4_K and Q6_K, K % 256 == 0
bool qgemv_kq_fast_shape_ok(int fmt, uint32_t rows, uint32_t k);  // same, without the pointer checks
cudaError_t launch_qgemv_kq_fast(int fmt, const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream);
void qgemv_q4k_fast_set_cta_cap(int cap);
// Kernel::MatMulId at decode sizes (1..8 tokens): every (token, slot) pair is a one-row GEMV against the
// matrix its expert id selects; a bad id sets status bit 128 (and reads expert 0 instead).
bool qgemv_kq_moe_shape_ok(int fmt, uint32_t tokens, uint32_t k);
cudaError_t launch_qgemv_kq_moe(int fmt, const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream);
// ---- qgemv_i8.cu: fast path for Int8 planes (K % 512 == 0); reads the activation planes
bool qgemv_i8_fast_shape_ok(uint32_t rows, uint32_t k);
cudaError_t launch_qgemv_i8_fast(const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream);  // tuning: at most this many CTAs per SM (0 = as many as fit)
cudaError_t launch_qgemv_i4_fast(const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream);  // Int4 nibble planes, same shapes

// out[bt, i, j] = 0 (+ extra) for the k == 0 case (crates/lapid-cpu/src/matmul/mod.rs:237-247).
cudaError_t launch_fill_zero_k(const GemvArgs &args, cudaStream_t stream);

// ---- qgemm_f32.cu
// Exact-f32 GEMM for more than 8 activation rows (rows = batch*m, flattened like GemvArgs).
struct GemmF32Args {
    const uint8_t *w;
    uint64_t scales_offset;
    const void *a;          // f32, f16 or bf16 rows (a_type), widened exactly to f32 as they are read
    int a_type;
    uint64_t a_off, a_bs, a_rs;
    float *out;
    uint64_t out_off, out_bs, out_rs;
    const float *extra;
    uint64_t ex_off;
    int64_t ex_s0, ex_s1, ex_s2;
    uint32_t rows, m, n, k;
    // Expert-indexed launches (moe.cu): rows = the tile space (64-row tiles), w = the expert stack
    const int32_t *tile_expert;  // nullptr for an ordinary launch
    const int32_t *row_pair;
    uint64_t id_stride;          // bytes between the experts' matrices
    uint32_t id_r;               // slots per token: pair p reads activation row p / id_r, writes output row p
    const uint8_t *iq_grid;      // i-quants: the format's codebook on this device (set by the launcher)
};
cudaError_t launch_qgemm_f32(int fmt, const GemmF32Args &args, cudaStream_t stream);

// ---- qgemm_tc.cu: tcgen05 tensor-core GEMM (Q4_K weights, bf16 operands, f32 accumulation)
struct GemmTcArgs {
    const uint8_t *w;
    const void *a;          // f32, f16 or bf16 rows (a_type); the kernel multiplies their bf16 roundings
    int a_type;
    uint64_t a_off, a_bs, a_rs;
    float *out;
    uint64_t out_off, out_bs, out_rs;
    const float *extra;
    uint64_t ex_off;
    int64_t ex_s0, ex_s1, ex_s2;
    uint32_t rows, m, n, k;
    int *status;
    float *partial;  // split-K launches: [splits][rows][n] partial sums in the scratch; nullptr otherwise
    // Expert-indexed launches (launch_qgemm_tc_moe): rows = the tile space, n = rows of ONE expert's matrix
    const int32_t *tile_expert;  // nullptr for an ordinary launch
    const int32_t *row_pair;
};
bool qgemm_tc_supported(int fmt, const GemmTcArgs &args);
size_t qgemm_tc_scratch_bytes(uint32_t rows, uint32_t n, uint32_t k, int sm_count);  // bf16 copy of the activations + split-K partial sums
void qgemm_tc_set_splitk(int v);  // tuning: -1 choose, 0 / 1 never, n > 1 always n ways
cudaError_t launch_qgemm_tc(int fmt, const GemmTcArgs &args, void *a_bf16_scratch, int sm_count, cudaStream_t stream, int *launched);
// Kernel::MatMulId on the tensor cores: `a_bf16` holds the activation rows in tile-space order (moe.cu), the
// weights are a dense stack of `experts` matrices [n, k] (no padding between them), mt in {64, 128, 256}.
bool qgemm_tc_moe_supported(int fmt, uint64_t experts, uint64_t n, uint64_t k, const void *w);
cudaError_t launch_qgemm_tc_moe(int fmt, const GemmTcArgs &args, uint32_t experts, uint32_t mt, void *a_bf16, cudaStream_t stream);
void qgemm_tc_set_wide(int v);  // tuning: -1 choose, 0 / 1 force one / two accumulators per CTA
void qgemm_tc_set_pair(int v);  // tuning: 1 = CTA pairs (cta_group::2) for the two-accumulator Q4_K tile
void qgemm_tc_set_tall(int v);  // tuning: -1 choose, 0 / 1 never / always 512 activation rows per CTA above 256 rows


// ---- moe.cu: device-side grouping of (token, slot) pairs by expert for Kernel::MatMulId
struct MoeRouteArgs {
    const int32_t *ids;  // [pairs]
    uint32_t pairs, experts, mt, max_tiles;
    int32_t *counts, *cursor, *offsets;  // [experts] each
    int32_t *tile_expert;                // [max_tiles]
    int32_t *row_pair;                   // [max_tiles * mt]
    int *status;
};
uint32_t moe_max_tiles(uint64_t pairs, uint64_t experts, uint32_t mt);
size_t moe_route_bytes(uint64_t pairs, uint64_t experts, uint32_t mt);
void moe_route_layout(void *scratch, uint64_t pairs, uint64_t experts, uint32_t mt, MoeRouteArgs &args);  // fills all but ids and status
cudaError_t launch_moe_route(const MoeRouteArgs &args, bool pdl, cudaStream_t stream);
cudaError_t launch_moe_gather_bf16(const float *x, const MoeRouteArgs &route, uint32_t r, uint32_t k, void *dst, cudaStream_t stream);

// ---- glue.cu: the row / elementwise steps between the projections of a layer (not on the matmul path)
struct RmsNormArgs {
    const TpPushTable *tp;  // not nullptr: x is the sum over ranks of what they pushed for the current call (x is ignored)
    int *status;
    uint32_t spin_limit;    // tp: polls of a peer's pair before the kernel gives up and sets status bit 64 (0 = the default)
    const float *x;         // [rows, cols]
    const float *residual;  // [rows, cols] added to x first, or nullptr
    const float *weight;    // [cols], or nullptr for a weight-less normalise
    float *sum_out;         // [rows, cols] receives x + residual, or nullptr
    float *out;             // [rows, cols]
    uint32_t rows, cols;
    float eps;
    ActOut q;               // q.qa set: `out` also goes out as a quantized activation operand (cols % 256 == 0)
};
bool rms_norm_shape_ok(uint32_t cols);  // multiple of 4, at most 16384
cudaError_t launch_rms_norm(const RmsNormArgs &args, bool pdl, cudaStream_t stream);
bool rms_norm_quant_ok(uint32_t cols);  // the row splits over the cluster in whole 32-element groups
// silu(gate) * up over [rows, cols] (q.qa set: also as a quantized activation operand; cols % 32 == 0)
cudaError_t launch_silu_mul(const float *gate, const float *up, float *out, uint64_t n, uint32_t cols, const ActOut &q, int sm_count,
                            bool pdl, cudaStream_t stream);

// ---- tp_allreduce.cu: one-shot all-reduce over peer-mapped memory
struct TpAllReduceArgs {
    void *peer[TP_MAX_RANKS];  // every rank's symmetric buffer as mapped on this GPU; peer[rank] is this rank's own
    int rank, world;
    uint64_t max_elems;        // f32 capacity of one slot
    float *data;               // local partial, replaced by the sum
    uint64_t count;            // multiple of 4, <= max_elems
    int *status;
    uint32_t spin_limit;       // polls of a peer's pair before the kernel gives up and sets status bit 64 (0 = the default)
    int push_only;             // 1: publish `data` to every rank's slots and return; the reader (tp rms_norm) sums and closes the call
};
size_t tp_comm_bytes(int world, uint64_t max_elems);
cudaError_t launch_tp_all_reduce(const TpAllReduceArgs &args, bool pdl, cudaStream_t stream);

}  // namespace lb

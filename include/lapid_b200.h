/*
 * lapid_b200.h -- C ABI of the B200 (sm_100a) backend for lapid's quantized matmul path.
 *
 * The library is a sibling of lapid-cuda: it implements the part of lapid's backend operator
 * surface that a `Kernel::MatMul` launch with a quantized, transposed B needs
 * (`lapid_compiler::Backend`, crates/lapid-compiler/src/backend.rs:8-63, and the MatMul launch
 * types of crates/lapid-compiler/src/ir.rs:226-282, :483-488), plus the lapid-quant byte-format
 * functions (crates/lapid-quant/src/lib.rs:97-160), behind plain C types so that a Rust
 * `impl Backend` can bind it with `extern "C"`.
 *
 * Conventions follow lapid-c (crates/lapid-c/src/error.rs:16-97, src/handle.rs:28-50):
 *  - every fallible function returns an int32 status, 0 = LAPID_B200_OK;
 *  - details of the last failure on the calling thread are a JSON object
 *    {"status": n, "error": "<lapid error code>", "message": "..."} from lapid_b200_last_error();
 *  - out-parameters come last and are untouched on failure;
 *  - handles are opaque and reference counted; *_retain / *_free accept NULL;
 *  - no exception or abort crosses the boundary; all functions are thread-safe. Launches on one
 *    device are serialised on that device's stream, as lapid-cuda does
 *    (crates/lapid-cuda/src/lib.rs:155-159).
 *
 * There is no CPU fallback: without a CUDA device every device function fails with
 * LAPID_B200_ERR_DEVICE_UNAVAILABLE.
 */
#ifndef LAPID_B200_H
#define LAPID_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define LAPID_B200_API __attribute__((visibility("default")))
#else
#define LAPID_B200_API
#endif

#define LAPID_B200_ABI_VERSION 1u

/* Status codes: the values of lapid-c's LAPID_ERR_* (crates/lapid-c/src/error.rs:16-36). */
typedef int32_t lapid_b200_status;
#define LAPID_B200_OK 0
#define LAPID_B200_ERR_INVALID_ARGUMENT 1
#define LAPID_B200_ERR_SHAPE_MISMATCH 2
#define LAPID_B200_ERR_UNSUPPORTED_DTYPE 3
#define LAPID_B200_ERR_NOT_FOUND 4
#define LAPID_B200_ERR_DEVICE_UNAVAILABLE 7
#define LAPID_B200_ERR_BACKEND 8          /* "cuda", "invalid_launch", "bad_launch" */
#define LAPID_B200_ERR_OUT_OF_MEMORY 9    /* "out_of_memory", "too_large" */
#define LAPID_B200_ERR_INDEX_OUT_OF_RANGE 10 /* "out_of_bounds", "index_out_of_range" */
#define LAPID_B200_ERR_ABI_MISMATCH 11
#define LAPID_B200_ERR_INTERNAL 13

/* Element type codes: lapid-c's LAPID_DTYPE_* (crates/lapid-c/src/lib.rs:37-60). INT8 is
 * lapid's plane layout of GGUF Q8_0 (crates/lapid-quant/src/lib.rs:5-17). */
#define LAPID_B200_DTYPE_F32 0
#define LAPID_B200_DTYPE_F16 1
#define LAPID_B200_DTYPE_BF16 2
#define LAPID_B200_DTYPE_I32 3
#define LAPID_B200_DTYPE_INT8 4
#define LAPID_B200_DTYPE_INT4 5
#define LAPID_B200_DTYPE_Q4_K 6
#define LAPID_B200_DTYPE_Q5_K 7
#define LAPID_B200_DTYPE_Q6_K 8
#define LAPID_B200_DTYPE_MXFP4 9 /* ggml block_mxfp4: 32 elements in 17 bytes (crates/lapid-quant/src/mxfp4.rs) */
/* ggml's grid-based i-quants, 256-element super-blocks stored as in GGUF (crates/lapid-c/src/lib.rs:53-60;
 * crates/lapid-quant/src/iq2.rs, iq3.rs): dequantize, from_ggml_blocks (blocks kept), Gather, MatMul and MatMulId.
 * lapid_b200_quantize answers `unsupported` for them. */
#define LAPID_B200_DTYPE_IQ2_XXS 10 /* 66-byte blocks, 2.0625 bits per weight */
#define LAPID_B200_DTYPE_IQ2_S 11   /* 82-byte blocks, 2.5625 */
#define LAPID_B200_DTYPE_IQ3_XXS 12 /* 98-byte blocks, 3.0625 */
#define LAPID_B200_DTYPE_IQ2_XS 13  /* 74-byte blocks, 2.3125 */
/* Not a lapid dtype: as a launch's a_dtype it says that input 0 is an activation operand already
 * quantized for this launch by lapid_b200_rms_norm_act / lapid_b200_silu_mul_act (see there). */
#define LAPID_B200_DTYPE_ACT_Q8 100

typedef struct lapid_b200_device lapid_b200_device;
typedef struct lapid_b200_buffer lapid_b200_buffer;

/* ---- library ------------------------------------------------------------------------- */
/* lapid_abi_version / lapid_check_abi (crates/lapid-c/src/lib.rs:110-125). */
LAPID_B200_API uint32_t lapid_b200_abi_version(void);
LAPID_B200_API lapid_b200_status lapid_b200_check_abi(uint32_t expected);
/* lapid_last_error (crates/lapid-c/src/error.rs:104-118): JSON of the calling thread's last
 * failure, valid until the next failing call on this thread; NULL when there was none. */
LAPID_B200_API const char *lapid_b200_last_error(void);

/* ---- device (Backend::name / device_name; `Device::cuda`, crates/lapid/src/device.rs) ---- */
/* Opens CUDA device `ordinal` (it must be compute capability 10.x) with its own stream. */
LAPID_B200_API lapid_b200_status lapid_b200_device_open(int32_t ordinal, lapid_b200_device **out);
LAPID_B200_API void lapid_b200_device_retain(lapid_b200_device *dev);
LAPID_B200_API void lapid_b200_device_free(lapid_b200_device *dev);
/* Backend::device_name: writes a NUL-terminated name, truncated to `cap` bytes. */
LAPID_B200_API lapid_b200_status lapid_b200_device_name(const lapid_b200_device *dev, char *out, size_t cap);
/* Makes later launches and copies of this device use `cuda_stream` (a cudaStream_t, e.g. the
 * stream of a framework that owns the surrounding work); NULL restores the device's own stream.
 * No counterpart in the reference, whose CUDA backend owns its single stream
 * (crates/lapid-cuda/src/execute.rs:1-3). */
LAPID_B200_API lapid_b200_status lapid_b200_device_set_stream(lapid_b200_device *dev, void *cuda_stream);
/* Waits for everything queued on the device's stream. */
LAPID_B200_API lapid_b200_status lapid_b200_device_synchronize(lapid_b200_device *dev);
/* Options, the counterpart of the reference's environment switches
 * (crates/lapid-cpu/src/matmul/mod.rs:52-57, crates/lapid-cuda/src/lib.rs:13-23):
 *   "gemv_max_rows" = "0".."8" (default 8, the reference's SMALL_M, crates/lapid-cpu/src/matmul/mod.rs:45):
 *                     launches with batch*m above it take the GEMM path;
 *   "gemm"          = "tc" (default): launches above gemv_max_rows with Q4_K, Q5_K or Q6_K weights (k a multiple
 *                     of 256) run on the tensor cores with bf16 operands (INT8 and INT4 use the exact kernel);
 *                     "f32": every such launch uses the exact-f32 kernel (lapid-cpu's qdeq numerics,
 *                     bit-identical to it);
 *   "gemv"          = "fast" (default) | "generic": specialised decode kernels where the shape allows;
 *   "act_reuse"     = "1" (default) | "0": share and hoist activation pre-passes inside a launch list;
 *   "pdl"           = "1" (default) | "0": programmatic dependent launch between the kernels of
 *                     a launch sequence (weights are staged while the producer still runs);
 *   "early_acts"    = "1" (default) | "0": decode launches whose activations were quantized by the
 *                     pre-pass at the head of the list read them, and compute their first results, before
 *                     the kernel in front of them has finished (they still write only after it has). */
LAPID_B200_API lapid_b200_status lapid_b200_device_set_option(lapid_b200_device *dev, const char *key, const char *value);

/* ---- buffers (Backend::alloc / upload / write / download, backend.rs:17-50) ------------- */
LAPID_B200_API lapid_b200_status lapid_b200_alloc(lapid_b200_device *dev, size_t bytes, lapid_b200_buffer **out);
LAPID_B200_API lapid_b200_status lapid_b200_upload(lapid_b200_device *dev, const void *host, size_t bytes, lapid_b200_buffer **out);
/* A buffer over device memory the caller owns (16-byte aligned, alive until the handle is
 * freed); the library never frees it. Counterpart of `map_host`'s "view without copying"
 * (backend.rs:21-26) for memory that is already on the device. */
LAPID_B200_API lapid_b200_status lapid_b200_wrap(lapid_b200_device *dev, void *device_ptr, size_t bytes, lapid_b200_buffer **out);
/* Overwrites bytes [offset, offset + bytes) from host memory; ordered before later launches. */
LAPID_B200_API lapid_b200_status lapid_b200_write(lapid_b200_buffer *buf, size_t offset, const void *host, size_t bytes);
/* Copies the first `bytes` bytes back to host memory after waiting for pending work. */
LAPID_B200_API lapid_b200_status lapid_b200_download(lapid_b200_buffer *buf, void *host, size_t bytes);
LAPID_B200_API void lapid_b200_buffer_retain(lapid_b200_buffer *buf);
LAPID_B200_API void lapid_b200_buffer_free(lapid_b200_buffer *buf);
LAPID_B200_API size_t lapid_b200_buffer_size(const lapid_b200_buffer *buf);
LAPID_B200_API void *lapid_b200_buffer_device_ptr(const lapid_b200_buffer *buf);

/* ---- launches (Kernel::MatMul, ir.rs:226-282; Launch, ir.rs:483-488) ---------------------- */
/* MatView (ir.rs:249-254): offsets and strides in ELEMENTS. */
typedef struct lapid_b200_matview {
    uint64_t offset, batch_stride, row_stride;
} lapid_b200_matview;

/* View of an epilogue extra over the rank-3 space [batch, m, n] (ir.rs `View`): element
 * (bt, i, j) at offset + bt*strides[0] + i*strides[1] + j*strides[2]; a bias over n is {0,0,1}. */
typedef struct lapid_b200_view3 {
    uint64_t offset;
    int64_t strides[3];
} lapid_b200_view3;

#define LAPID_B200_KERNEL_MATMUL 2 /* position of MatMul in `enum Kernel`, ir.rs:395-414 */
/* Kernel::Gather (ir.rs:284-300, CPU crates/lapid-cpu/src/rows.rs:164-215): out[i, :] = dequant(table[ids[i], :]),
 * the embedding lookup from a quantized table. In a launch of this kind: b_dtype = table dtype (F32,
 * INT8, INT4, Q4_K, Q5_K, Q6_K), out_dtype F32, k = rows of the table, n = cols, m = count, batch 1;
 * inputs = {table [k, n] in lapid-quant layout, indices i32 [m] contiguous}, n_inputs 2; output f32
 * [m, n] contiguous (the views are not used). An index outside [0, k) makes execute fail with
 * "index_out_of_range" after the launch sequence ran; the kernel does not read out of bounds. */
#define LAPID_B200_KERNEL_GATHER 3
/* Kernel::MatMulId (ir.rs:425-443, CPU crates/lapid-cpu/src/moe.rs:21-120): the mixture-of-experts matmul
 * out[t, s, :] = W[ids[t, s]] x[t] over a stack of e quantized matrices [n, k], each a lapid-quant matrix at
 * byte offset expert * layout(n, k).total. In a launch of this kind: b_dtype = w dtype (INT8, INT4, Q4_K, Q5_K, Q6_K),
 * a_dtype and out_dtype F32, m = t (tokens), batch = r (slots per token), b.batch_stride = e, n, k;
 * inputs = {x f32 [t, k] contiguous, w, ids i32 [t, r] contiguous}, n_inputs 3; output f32 [t, r, n]
 * contiguous (the other view fields are not used). t <= 8 uses the int8-activation arithmetic of the decode
 * path for every pair, more tokens the prefill arithmetic (as lapid-cpu: float activations when t > 8,
 * moe.rs:107-109). An id outside [0, e) makes execute fail with "index_out_of_range" after the launch
 * sequence ran; the kernels do not read out of bounds. */
#define LAPID_B200_KERNEL_MATMUL_ID 4

/* Fused epilogues (MatMulSpec.epilogue, ir.rs:234-247; the expression type: ir.rs:94-111). NONE and ADD
 * (`Load(0) + Load(1)`) are the two shapes lapid's lowering emits for projections
 * (crates/lapid-compiler/src/lower/emit.rs:199-262). EXPR is any f32 expression over Load(0) = the accumulator and
 * Load(1) = extras[0] (n_inputs 3 when the program loads it, else 2), given in postfix order in `expr[0 .. n_expr)`:
 * one word per node, `op | arg << 8`; LAPID_B200_EXPR_CONST is followed by a word with the constant's bits. It is what
 * the elementwise chain behind a projection lowers to -- silu(acc) for the gate of a gated MLP, acc * extras[0] for
 * its up projection (crates/lapid-nn/src/mlp.rs:84), so that no elementwise kernel is left between gate/up and down.
 * At most 24 words and four values on the evaluation stack; the integer nodes of the reference's expression type
 * (LoadBits, IntUnary, IntBinary, Convert) answer "unsupported". Decode kernels evaluate it in their stores; a
 * prefill launch applies it to its output in place with one more kernel. Transcendental nodes are CUDA's f32
 * functions: they agree with lapid-cpu's own polynomials to a few ulp, not bit for bit. */
#define LAPID_B200_EPILOGUE_NONE 0
#define LAPID_B200_EPILOGUE_ADD 1
#define LAPID_B200_EPILOGUE_EXPR 2
#define LAPID_B200_EXPR_WORDS 24
#define LAPID_B200_EXPR_LOAD 1   /* arg: 0 = accumulator, 1 = extras[0] */
#define LAPID_B200_EXPR_CONST 2  /* next word: f32 bits */
/* UnaryOp (crates/lapid-tensor/src/op.rs:11-23), in its order, from 16 */
#define LAPID_B200_EXPR_NEG 16
#define LAPID_B200_EXPR_EXP 17
#define LAPID_B200_EXPR_LOG 18
#define LAPID_B200_EXPR_SQRT 19
#define LAPID_B200_EXPR_RSQRT 20
#define LAPID_B200_EXPR_RECIP 21
#define LAPID_B200_EXPR_SIN 22
#define LAPID_B200_EXPR_COS 23
#define LAPID_B200_EXPR_TANH 24
#define LAPID_B200_EXPR_ERF 25
#define LAPID_B200_EXPR_ABS 26
/* the float BinaryOps (op.rs:26-37), in their order, from 32: pops b then a, pushes a op b */
#define LAPID_B200_EXPR_ADD 32
#define LAPID_B200_EXPR_SUB 33
#define LAPID_B200_EXPR_MUL 34
#define LAPID_B200_EXPR_DIV 35
#define LAPID_B200_EXPR_MAX 36
#define LAPID_B200_EXPR_MIN 37
#define LAPID_B200_EXPR_POW 38
#define LAPID_B200_EXPR_CMPLT 39
#define LAPID_B200_EXPR_CMPEQ 40
#define LAPID_B200_EXPR_WHERE 48 /* pops b, a, cond; pushes cond != 0 ? a : b */

typedef struct lapid_b200_launch {
    int32_t kind;         /* LAPID_B200_KERNEL_MATMUL (the fields below describe it), LAPID_B200_KERNEL_GATHER or LAPID_B200_KERNEL_MATMUL_ID (see above) */
    int32_t a_dtype;      /* MatMulSpec.a_dtype: F32, F16 or BF16 -- half types are widened exactly to f32 as they are read, as
                             lapid-cpu's load_contig does (crates/lapid-cpu/src/matmul/mod.rs:165-286) -- or LAPID_B200_DTYPE_ACT_Q8 (above) */
    int32_t b_dtype;      /* MatMulSpec.b_dtype: INT8 | INT4 | Q4_K | Q5_K | Q6_K | MXFP4 | IQ2_XXS | IQ2_XS | IQ2_S | IQ3_XXS */
    int32_t out_dtype;    /* MatMulSpec.out_dtype: F32 */
    int32_t b_transposed; /* must be 1 for a quantized B */
    int32_t epilogue;     /* LAPID_B200_EPILOGUE_* */
    int32_t extra_dtype;  /* dtype of extras[0] when the epilogue reads it: F32 */
    int32_t n_inputs;     /* 2, or 3 with an extra */
    uint64_t batch, m, n, k;         /* MatMulDims */
    lapid_b200_matview a, b, out;    /* b: offset 0, batch_stride 0 (quantized B, ir.rs:232-233) */
    lapid_b200_view3 extra;          /* MatMulDims.extra_views[0] */
    uint32_t inputs[3];   /* BufIds: a, b, extras[0] -- indices into `buffers` of execute */
    uint32_t output;      /* BufId of the output */
    uint32_t n_expr;      /* epilogue == EXPR: words of the program */
    uint32_t expr[LAPID_B200_EXPR_WORDS];
} lapid_b200_launch;

/* Backend::prepare (backend.rs:51-54): validates the launches and sizes the device's scratch so
 * that `execute` allocates nothing afterwards. Optional; execute also works cold. */
LAPID_B200_API lapid_b200_status lapid_b200_prepare(lapid_b200_device *dev, const lapid_b200_launch *launches, size_t n_launches);
/* Backend::execute (backend.rs:55-58): runs the launches in order and waits; launch k+1 sees
 * all writes of launch k; `buffers[id]` is the buffer of BufId `id` (ids may alias). */
LAPID_B200_API lapid_b200_status lapid_b200_execute(lapid_b200_device *dev, const lapid_b200_launch *launches, size_t n_launches,
                                     lapid_b200_buffer *const *buffers, size_t n_buffers);
/* Same, but returns once the work is queued on the device's stream (for callers that run a whole
 * token in one stream or capture it in a CUDA graph). Call prepare first when capturing. No
 * counterpart in the reference, whose execute always waits. */
LAPID_B200_API lapid_b200_status lapid_b200_execute_async(lapid_b200_device *dev, const lapid_b200_launch *launches,
                                           size_t n_launches, lapid_b200_buffer *const *buffers, size_t n_buffers);

/* One decode step with host buffers as ONE call: Backend::write of the step's inputs, Backend::execute and
 * Backend::read of its results (backend.rs:36-58), pipelined. The launches run in consecutive chunks of
 * `chunk_launches` (0: the library picks up to three chunks that carry about the same number of transferred bytes); every write is uploaded on a copy stream of its own just before the
 * chunk that holds the launch it names (`launch`: the FIRST launch that reads what it brings), every read is
 * downloaded on a second copy stream right after the chunk that holds the launch it names (`launch`: the LAST launch
 * that writes what it takes), so that uploads, launches and downloads of different chunks overlap (the two copy
 * engines and the SMs at the same time). The result is that of all writes, execute, all reads in that order; the
 * call returns when everything has finished. Declarations are checked against the launches' views: a write whose
 * memory an earlier chunk uses, or a read whose memory a later chunk writes, is `invalid_launch`. Host memory
 * should be page-locked (pageable memory is staged by the driver and overlaps nothing). Not for use inside a
 * stream capture. */
typedef struct lapid_b200_io {
    uint32_t buffer; /* index into the call's buffers */
    uint32_t launch; /* index into the call's launches (see above) */
    uint64_t offset; /* bytes from the start of the buffer */
    void *host;      /* source of a write, destination of a read */
    uint64_t bytes;
} lapid_b200_io;
LAPID_B200_API lapid_b200_status lapid_b200_execute_io(lapid_b200_device *dev, const lapid_b200_launch *launches, size_t n_launches,
                                        lapid_b200_buffer *const *buffers, size_t n_buffers, const lapid_b200_io *writes, size_t n_writes,
                                        const lapid_b200_io *reads, size_t n_reads, size_t chunk_launches);
/* Number of kernels this library launched on `dev` since the last call. */
LAPID_B200_API uint64_t lapid_b200_take_launch_count(lapid_b200_device *dev);
/* Backend::take_profile (backend.rs:59-62; CUDA side crates/lapid-cuda/src/execute.rs:45-76): GPU time per kernel kind
 * -- "matmul_decode", "matmul_prefill", "gather", "matmul_id" -- accumulated since the last call while the device option
 * "profile" is "1" (every launch of an execute list is then bracketed by events and runs on its own: nothing is
 * grouped, and execute_async waits like execute), sorted by time, then cleared. Writes all *n entries when
 * cap >= *n, else only sets *n so that the caller can come back with room (nothing is cleared then). */
typedef struct lapid_b200_profile_entry {
    char kind[24];
    uint64_t launches;
    double ms;
} lapid_b200_profile_entry;
LAPID_B200_API lapid_b200_status lapid_b200_take_profile(lapid_b200_device *dev, lapid_b200_profile_entry *entries, size_t cap, size_t *n);
/* Diagnostics of the balanced-stream decode kernel (no counterpart in the reference): record, for the next
 * `launches` launches of that kernel on this process, one row of 16 words per CTA -- [0] entry time (ns, global
 * timer), then SM clock cycles at [1] entry, [2] first loads issued, [3] first data there, [4] before and [5] after
 * the wait for the kernel in front, [6] exit; [7] exit time (ns); [8] SM; [9] work units; [10] cycles its first warp
 * waited for data. `read` copies launches x ctas x 16 words (launch order) and says how many launches were recorded
 * and how many CTA rows each launch has (rows of CTAs that did not exist are zero). begin(0) frees the buffer. */
LAPID_B200_API lapid_b200_status lapid_b200_decode_trace_begin(lapid_b200_device *dev, uint32_t launches);
LAPID_B200_API lapid_b200_status lapid_b200_decode_trace_read(lapid_b200_device *dev, uint64_t *out, uint64_t cap_words,
                                                               uint32_t *launches, uint32_t *ctas);

/* ---- lapid-quant surface (crates/lapid-quant/src/lib.rs:84-160) ---------------------------- */
typedef struct lapid_b200_layout {
    uint64_t rows, cols, qs_offset, qs_bytes, scales_offset, scales_bytes, total;
} lapid_b200_layout;
/* `layout(format, rows, cols)` (lib.rs:97-125). Host only; needs no device. */
LAPID_B200_API lapid_b200_status lapid_b200_quant_layout(int32_t format, uint64_t rows, uint64_t cols, lapid_b200_layout *out);
/* `dequantize` (lib.rs:136-139) on the device: src holds a quantized [rows, cols] matrix, dst
 * receives rows*cols f32, bit-identical to lapid-quant's values. */
LAPID_B200_API lapid_b200_status lapid_b200_dequantize(lapid_b200_device *dev, int32_t format, const lapid_b200_buffer *src,
                                        uint64_t rows, uint64_t cols, lapid_b200_buffer *dst);
/* `quantize` (lib.rs:131-133) on the device: src holds rows*cols f32, dst receives layout.total
 * bytes, byte-identical to lapid-quant's output (padding zeroed). */
LAPID_B200_API lapid_b200_status lapid_b200_quantize(lapid_b200_device *dev, int32_t format, const lapid_b200_buffer *src,
                                      uint64_t rows, uint64_t cols, lapid_b200_buffer *dst);
/* `from_ggml_blocks` (lib.rs:147-149): GGUF blocks (`src_bytes` of them in src) -> lapid layout. */
LAPID_B200_API lapid_b200_status lapid_b200_from_ggml_blocks(lapid_b200_device *dev, int32_t format, const lapid_b200_buffer *src,
                                              uint64_t src_bytes, uint64_t rows, uint64_t cols,
                                              lapid_b200_buffer *dst);

/* ---- tensor parallelism (no counterpart in the reference, which has no multi-GPU code) -------- */
/* One-shot all-reduce (f32 sum, in place) of a row-parallel projection's partial results over up to
 * 8 GPUs of one NVLink domain, through peer-mapped memory instead of a library collective.
 * The caller (one process per GPU) allocates, on every rank, one zero-filled buffer of
 * lapid_b200_tp_comm_bytes(world, max_elems) bytes that every peer can address ("symmetric
 * memory": cuMemMap / IPC mappings, e.g. torch.distributed._symmetric_memory), and passes the
 * `world` base addresses as mapped on THIS GPU, its own at index `rank`. All ranks must issue the
 * same sequence of all-reduce calls. Sums are formed in rank order on every rank, so the result is
 * bit-identical on all ranks. Waits on peers are bounded (status "backend" at the next execute). */
typedef struct lapid_b200_tp_comm lapid_b200_tp_comm;
LAPID_B200_API uint64_t lapid_b200_tp_comm_bytes(int32_t world, uint64_t max_elems);
LAPID_B200_API lapid_b200_status lapid_b200_tp_comm_create(lapid_b200_device *dev, int32_t rank, int32_t world,
                                                           void *const *peer_bases, uint64_t max_elems,
                                                           lapid_b200_tp_comm **out);
LAPID_B200_API void lapid_b200_tp_comm_free(lapid_b200_tp_comm *comm);
/* Queues the all-reduce of `count` f32 (multiple of 4, <= max_elems) at element `offset` of `data`
 * on the device's stream; returns without waiting. */
LAPID_B200_API lapid_b200_status lapid_b200_tp_all_reduce(lapid_b200_tp_comm *comm, lapid_b200_buffer *data,
                                                          uint64_t offset, uint64_t count);

/* The all-reduce of a decode step without a kernel of its own: the row-parallel projection hands its
 * partial to every rank from the GEMV's epilogue, and the normalisation that follows polls and sums
 * the ranks' partials itself (in rank order: bit-identical on every rank).
 *   lapid_b200_tp_matmul_push: ONE decode MatMul launch (batch*m in 1..8, contiguous output view,
 *     rows*n a multiple of 4 and <= max_elems). Launches that take a K-quant fast kernel push from
 *     the kernel; others run as usual and a small kernel publishes their output buffer. The output
 *     buffer of a pushing launch is not written.
 *   lapid_b200_tp_rms_norm: lapid_b200_rms_norm (below) with x = the sum over ranks of the partials of
 *     the push in progress, [rows, cols] row-major; closes the call. Every push must be followed by
 *     exactly one lapid_b200_tp_rms_norm on every rank before the next push or all-reduce on this
 *     comm. */
LAPID_B200_API lapid_b200_status lapid_b200_tp_matmul_push(lapid_b200_tp_comm *comm, const lapid_b200_launch *launch,
                                                           lapid_b200_buffer *const *buffers, size_t n_buffers);
LAPID_B200_API lapid_b200_status lapid_b200_tp_rms_norm(lapid_b200_tp_comm *comm, lapid_b200_buffer *residual,
                                                        lapid_b200_buffer *weight, lapid_b200_buffer *sum_out,
                                                        lapid_b200_buffer *out, uint64_t rows, uint64_t cols, float eps);

/* ---- the steps between the projections of a layer ------------------------------------------- */
/* Not part of the quantized-matmul path: two small kernels so that a layer-stack measurement is not
 * dominated by a framework's elementwise launches. Queued on the device's stream, not waited for.
 *
 * lapid_b200_rms_norm: lapid's Kernel::RmsNorm (crates/lapid-compiler/src/ir.rs:407-409, CPU
 *   crates/lapid-cpu/src/rows.rs:118-156) with the residual add that precedes it folded in:
 *     h = x (+ residual);  out = h * rsqrt(mean(h*h) + eps) (* weight);  sum_out = h   (if given)
 *   x, residual, sum_out, out: [rows, cols] f32 contiguous; weight: [cols] f32. residual, weight and
 *   sum_out may be NULL. cols: multiple of 4, at most 16384. sum_out may be x or residual (in place).
 * lapid_b200_silu_mul: out = gate / (1 + exp(-gate)) * up over `count` f32 (multiple of 4), the SwiGLU
 *   product (crates/lapid-nn/src/mlp.rs:84), an Elementwise kernel in lapid. out may be gate or up. */
LAPID_B200_API lapid_b200_status lapid_b200_rms_norm(lapid_b200_device *dev, lapid_b200_buffer *x, lapid_b200_buffer *residual,
                                                     lapid_b200_buffer *weight, lapid_b200_buffer *sum_out,
                                                     lapid_b200_buffer *out, uint64_t rows, uint64_t cols, float eps);
LAPID_B200_API lapid_b200_status lapid_b200_silu_mul(lapid_b200_device *dev, lapid_b200_buffer *gate, lapid_b200_buffer *up,
                                                     lapid_b200_buffer *out, uint64_t count);

/* ---- producers that quantize for the projection that follows (RMSNorm + activation-quant prologue) */
/* A decode launch (batch*m <= 8) multiplies int8-quantized activation rows; by default `execute` makes
 * them from the f32 operand with a small pre-pass kernel per distinct operand. The `_act` forms of the
 * glue kernels write their result in that quantized form as well (same arithmetic, bit for bit), and a
 * launch with a_dtype = LAPID_B200_DTYPE_ACT_Q8 and input 0 = that buffer skips its pre-pass.
 *   lapid_b200_act_layout: for a decode MatMul launch (a_dtype F32 or ACT_Q8), the layout code its kernel
 *     reads and the bytes of the quantized operand; fails with "invalid_launch" for other launches.
 *     Launches with the same (layout, batch*m, k) can share one quantized operand (q/k/v; gate/up).
 *   *_act: as the plain forms, plus `qact` (>= the bytes above, 16-byte aligned) written in `layout`;
 *     rows*cols of the producer = batch*m and k of the consumer; cols a multiple of 256 (rms_norm:
 *     up to 16384 and cols/32 a multiple of its cluster size, which holds for multiples of 1024).
 *     qact NULL: exactly the plain form. */
LAPID_B200_API lapid_b200_status lapid_b200_act_layout(lapid_b200_device *dev, const lapid_b200_launch *launch, int32_t *layout,
                                                       uint64_t *bytes);
/* The pre-pass as a call of its own: `quantize_row_sums` (crates/lapid-cpu/src/matmul/quant.rs:30-89) for `rows`
 * (1..8) contiguous f32 rows of `k` elements in `a`, written to `qact` in `layout` (0: planes -- int8 q[rows][k],
 * then at the next multiple of 256 bytes f32 d[rows][k/32], then likewise f32 d*sum(q)[rows][k/32]; 1 and 2: the
 * record and tile layouts of the specialised decode kernels, k a multiple of 256). Per 32-element group:
 * amax = max|x|, d = amax/127, id = d > 0 ? 1/d : 0, q = clamp(round_half_even(x*id), -127, 127). Queued on the
 * device's stream, not waited for. A launch with a_dtype ACT_Q8 whose lapid_b200_act_layout matches reads it. */
LAPID_B200_API lapid_b200_status lapid_b200_quantize_activations(lapid_b200_device *dev, const lapid_b200_buffer *a, uint64_t rows,
                                                                 uint64_t k, int32_t layout, lapid_b200_buffer *qact);
LAPID_B200_API lapid_b200_status lapid_b200_rms_norm_act(lapid_b200_device *dev, lapid_b200_buffer *x, lapid_b200_buffer *residual,
                                                         lapid_b200_buffer *weight, lapid_b200_buffer *sum_out,
                                                         lapid_b200_buffer *out, uint64_t rows, uint64_t cols, float eps,
                                                         lapid_b200_buffer *qact, int32_t layout);
LAPID_B200_API lapid_b200_status lapid_b200_tp_rms_norm_act(lapid_b200_tp_comm *comm, lapid_b200_buffer *residual,
                                                            lapid_b200_buffer *weight, lapid_b200_buffer *sum_out,
                                                            lapid_b200_buffer *out, uint64_t rows, uint64_t cols, float eps,
                                                            lapid_b200_buffer *qact, int32_t layout);
LAPID_B200_API lapid_b200_status lapid_b200_silu_mul_act(lapid_b200_device *dev, lapid_b200_buffer *gate, lapid_b200_buffer *up,
                                                         lapid_b200_buffer *out, uint64_t rows, uint64_t cols,
                                                         lapid_b200_buffer *qact, int32_t layout);

/* ---- decode without allocation ------------------------------------------------------------ */
/* This entry point has no counterpart in the reference. It exists for hosts that may not allocate
 * device memory when they need a matvec (an engine that gave all device memory to its own arena at
 * start-up, a loop with a fixed memory budget, a plug-in living under another runtime's
 * allocator): it makes no cudaMalloc / cudaFree or other allocating call on any path, because the
 * quantized activations go to an array inside the library image instead of a grown scratch block.
 *
 *   out[r, j] = sum_k a[r, k] * dequant(w)[j, k]     r < rows (1..8), j < n, k % 256 == 0
 *
 * a (rows x k f32, contiguous), w (Q4_K [n, k], 16-byte aligned, w_bytes readable) and out
 * (rows x n f32, contiguous) are DEVICE pointers on device `ordinal`, owned by the caller; the work
 * is queued on `cuda_stream` (NULL = the legacy default stream) and not waited for. Same arithmetic
 * as a MatMul launch with batch*m <= 8 through lapid_b200_execute.
 * Limits and rules: rows * k <= 65536 (the array holds LAPID_B200_STATIC_SCRATCH_BYTES; a larger
 * request fails with "too_large"); every GPU that loads the library carries the array until exit;
 * all calls on a GPU share it and it keeps the previous call's contents (nothing in it needs
 * clearing), so calls that can overlap on the GPU race -- keep them on one stream or order them
 * with events; the first call on a GPU also looks up the array's address, and the first call on a GPU
 * with a given (rows, k) configures that kernel variant, so make those calls before any stream capture.
 * The calling thread's current device is put back before the call returns. A device-side wait that gave
 * up (the result is then wrong) is not reported by this call, which does not wait: read it with
 * lapid_b200_gemv_q4k_static_status after synchronising. */
#define LAPID_B200_STATIC_SCRATCH_BYTES 86016u
LAPID_B200_API lapid_b200_status lapid_b200_gemv_q4k_static(int32_t ordinal, void *cuda_stream, const float *a, const void *w,
                                                            uint64_t w_bytes, float *out, uint32_t rows, uint32_t n, uint32_t k);
/* Companion of the call above (no counterpart in the reference either): writes to *out, and clears, the word in
 * which the static path's kernels on GPU `ordinal` record a bounded wait that gave up (0 = none since the last
 * read; nonzero = the outputs of the calls since then are invalid). Synchronise the stream(s) those calls were
 * queued on first. Allocates nothing. */
LAPID_B200_API lapid_b200_status lapid_b200_gemv_q4k_static_status(int32_t ordinal, int32_t *out);

#ifdef __cplusplus
}
#endif
#endif /* LAPID_B200_H */

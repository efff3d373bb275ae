// Host side of the library: the device / buffer objects behind the C handles, launch
// validation and dispatch, and the extern "C" entry points declared in lapid_b200.h.
//
// It mirrors, for the quantized-matmul path only:
//   Backend::{alloc, upload, write, download, prepare, execute}  crates/lapid-compiler/src/backend.rs:8-63
//   launch validation of matmul::run                             crates/lapid-cpu/src/matmul/mod.rs:165-262
//   buffer-id and aliasing checks of run_launch                  crates/lapid-cpu/src/lib.rs:380-397
//   QMat::new (shape and size checks of the quantized operand)   crates/lapid-cpu/src/qmat.rs:38-60
//   status codes, last-error JSON, panic guard                   crates/lapid-c/src/error.rs:16-97
#include "../../include/lapid_b200.h"

#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <map>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "kernels.h"

namespace {

// ------------------------------------------------------------------ errors
struct Error {
    const char *code;  // lapid's `Error::code` strings
    std::string message;
};

[[noreturn]] void fail(const char *code, std::string msg) { throw Error{code, std::move(msg)}; }

// crates/lapid-c/src/error.rs:49-66
int32_t status_of(const char *code) {
    auto is = [&](const char *s) { return std::strcmp(code, s) == 0; };
    if (is("invalid_argument")) return LAPID_B200_ERR_INVALID_ARGUMENT;
    if (is("shape_mismatch")) return LAPID_B200_ERR_SHAPE_MISMATCH;
    if (is("unsupported_dtype") || is("unsupported")) return LAPID_B200_ERR_UNSUPPORTED_DTYPE;
    if (is("not_found")) return LAPID_B200_ERR_NOT_FOUND;
    if (is("device_unavailable") || is("cuda_unavailable")) return LAPID_B200_ERR_DEVICE_UNAVAILABLE;
    if (is("backend") || is("cuda") || is("invalid_launch") || is("bad_launch") || is("wrong_backend") ||
        is("buffer_aliasing") || is("read_only_buffer"))
        return LAPID_B200_ERR_BACKEND;
    if (is("out_of_memory") || is("too_large")) return LAPID_B200_ERR_OUT_OF_MEMORY;
    if (is("index_out_of_range") || is("out_of_bounds")) return LAPID_B200_ERR_INDEX_OUT_OF_RANGE;
    if (is("abi_mismatch")) return LAPID_B200_ERR_ABI_MISMATCH;
    return LAPID_B200_ERR_INTERNAL;
}

thread_local std::string g_last_error;
thread_local bool g_has_error = false;

std::string json_escape(const std::string &s) {
    std::string o;
    for (unsigned char c : s) {
        if (c == '"' || c == '\\') {
            o += '\\';
            o += (char)c;
        } else if (c < 0x20) {
            char buf[8];
            std::snprintf(buf, sizeof buf, "\\u%04x", c);
            o += buf;
        } else {
            o += (char)c;
        }
    }
    return o;
}

int32_t record(const Error &e) {
    int32_t st = status_of(e.code);
    g_last_error = "{\"status\": " + std::to_string(st) + ", \"error\": \"" + json_escape(e.code) + "\", \"message\": \"" +
                   json_escape(e.message) + "\"}";
    g_has_error = true;
    return st;
}

template <class F> int32_t guard(F &&f) {
    try {
        f();
        return LAPID_B200_OK;
    } catch (const Error &e) {
        return record(e);
    } catch (const std::bad_alloc &) {
        return record(Error{"out_of_memory", "host allocation failed"});
    } catch (const std::exception &e) {
        return record(Error{"panic", e.what()});
    } catch (...) {
        return record(Error{"panic", "unknown exception"});
    }
}

void cuda_check(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return;
    const char *code = (e == cudaErrorMemoryAllocation) ? "out_of_memory" : "cuda";
    fail(code, std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")");
}

// ------------------------------------------------------------------ layout (lapid-quant lib.rs:84-125)
// the grid-based i-quants (crates/lapid-quant/src/lib.rs:79-82)
bool is_iquant(int32_t dt) {
    return dt == LAPID_B200_DTYPE_IQ2_XXS || dt == LAPID_B200_DTYPE_IQ2_XS || dt == LAPID_B200_DTYPE_IQ2_S || dt == LAPID_B200_DTYPE_IQ3_XXS;
}
bool is_quant(int32_t dt) {
    return dt == LAPID_B200_DTYPE_INT8 || dt == LAPID_B200_DTYPE_INT4 || dt == LAPID_B200_DTYPE_Q4_K || dt == LAPID_B200_DTYPE_Q5_K ||
           dt == LAPID_B200_DTYPE_Q6_K || dt == LAPID_B200_DTYPE_MXFP4 || is_iquant(dt);
}
bool is_act_float(int32_t dt) { return dt == LAPID_B200_DTYPE_F32 || dt == LAPID_B200_DTYPE_F16 || dt == LAPID_B200_DTYPE_BF16; }
// ACT_F32 / ACT_F16 / ACT_BF16 of the kernels, and the element size, for a launch's a_dtype
int act_type_of(int32_t dt) { return dt == LAPID_B200_DTYPE_F16 ? 1 : dt == LAPID_B200_DTYPE_BF16 ? 2 : 0; }
uint64_t act_elem_size(int32_t dt) { return dt == LAPID_B200_DTYPE_F32 ? 4 : 2; }
bool has_min_term(int32_t dt) { return dt == LAPID_B200_DTYPE_Q4_K || dt == LAPID_B200_DTYPE_Q5_K; }  // the decode tiles need d * sum(q) per activation group
uint64_t block_elems(int32_t dt) { return (dt == LAPID_B200_DTYPE_INT8 || dt == LAPID_B200_DTYPE_INT4 || dt == LAPID_B200_DTYPE_MXFP4) ? 32 : 256; }
uint64_t block_bytes(int32_t dt) {  // array-of-structs formats (lib.rs:62-75); 0 for the plane formats
    switch (dt) {
        case LAPID_B200_DTYPE_Q4_K: return 144;
        case LAPID_B200_DTYPE_Q5_K: return 176;
        case LAPID_B200_DTYPE_Q6_K: return 210;
        case LAPID_B200_DTYPE_MXFP4: return 17;
        case LAPID_B200_DTYPE_IQ2_XXS: return 66;
        case LAPID_B200_DTYPE_IQ2_XS: return 74;
        case LAPID_B200_DTYPE_IQ2_S: return 82;
        case LAPID_B200_DTYPE_IQ3_XXS: return 98;
        default: return 0;
    }
}
uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

lapid_b200_layout layout_of(int32_t fmt, uint64_t rows, uint64_t cols) {
    if (!is_quant(fmt)) fail("unsupported_dtype", "dtype " + std::to_string(fmt) + " is not a supported quantized format");
    uint64_t be = block_elems(fmt);
    if (cols % be != 0)
        fail("invalid_launch", "quantized matrix cols " + std::to_string(cols) + " not a multiple of " + std::to_string(be));
    if (cols != 0 && rows > UINT64_MAX / 2 / cols) fail("too_large", "quantized matrix size overflows");
    lapid_b200_layout l{};
    l.rows = rows;
    l.cols = cols;
    if (block_bytes(fmt)) {
        uint64_t n = rows * (cols / be) * block_bytes(fmt);
        l.qs_offset = 0;
        l.qs_bytes = n;
        l.scales_offset = n;
        l.scales_bytes = 0;
        l.total = align_up(n, 256);
        return l;
    }
    l.qs_offset = 0;
    l.qs_bytes = fmt == LAPID_B200_DTYPE_INT4 ? rows * cols / 2 : rows * cols;  // Int4: two elements of a group per byte
    l.scales_offset = align_up(l.qs_bytes, 256);
    l.scales_bytes = rows * (cols / 32) * 2;
    l.total = align_up(l.scales_offset + l.scales_bytes, 256);
    return l;
}

}  // namespace

// ------------------------------------------------------------------ handles
struct lapid_b200_device {
    std::atomic<int> refs{1};
    int ordinal = 0;
    int sm_count = 0;
    std::string name;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    // execute_io: the copy streams (one per direction: the two copy engines run at the same time) and one event per chunk
    cudaStream_t io_in = nullptr, io_out = nullptr;
    std::vector<cudaEvent_t> io_events;
    std::mutex mu;  // serialises launches, like lapid-cuda's mutex-guarded Exec
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    std::atomic<uint64_t> launches{0};
    int *status_host = nullptr;  // pinned, mapped: kernels report a bounded wait that gave up here
    int *status_dev = nullptr;
    bool pdl = true;
    uint32_t gemv_max_rows = 8;
    // Inside one execute list: kernels launched since the batched activation pre-pass at its head, -1 when the list
    // has none. The first kernel after that pre-pass is launched fully serialised (no programmatic dependent
    // launch), so every later kernel of the list starts after the pre-pass has completed and may read its
    // results before its own dependency wait (GemvArgs::early).
    int after_hoist = -1;
    bool early_acts = true;  // option "early_acts"
    uint32_t tp_spin_limit = 0;  // option "tp_spin_limit": polls before a tensor-parallel wait gives up (0 = the kernels' default)
    bool pdl_launch() {
        const bool p = pdl && after_hoist != 0;
        if (after_hoist >= 0) after_hoist++;
        return p;
    }
    bool early_ok(bool hoisted) const { return early_acts && pdl && hoisted && after_hoist >= 1; }
    bool act_reuse = true;  // share / hoist activation pre-passes inside one launch list
    bool gemv_fast = true;   // specialised GEMV kernels where the shape allows; off = generic kernel only
    bool gemv_group = true;  // consecutive independent K-quant decode launches of one list share a kernel
    uint32_t gemv_mma_rows = 2;  // Q4_K decode launches with at least this many rows use the int8 tensor-core kernel; 0 = never
    // balanced-stream tensor-core decode kernel (qgemv_kq_stream.cu): 0 never; 1 (default) Q5_K always and Q4_K where
    // it is the faster one (launch_qgemv_q4k_mma decides); 2 both formats always
    int gemv_stream = 1;
    // MXFP4 decode launches with at least this many rows use the int8 tensor-core kernel (0 = never): about 18.5 us on
    // 14336 x 4096 whatever the row count, against 15.8 / 17.9 / 25.4 / 42.9 us of the dp4a kernel at 1 / 2 / 4 / 8 rows
    uint32_t mxfp4_mma_rows = 3;
    bool small_dp4a = true;  // small Q5_K / Q6_K matrices at 3 and 4 rows on the dp4a kernel (see plan_launch)
    bool two_row_dp4a = false;    // two early Q4_K rows on the dp4a kernel (see execute_impl)
    lb::StreamWs stream_ws{};    // workspace of that kernel: partial sums in flight between CTAs (all zero between launches)
    bool gemm_f32 = false;  // true: rows > gemv_max_rows always take the exact-f32 GEMM instead of the tensor cores
    // option "profile": every launch of an execute list is bracketed by events (launches run one by one then: nothing is
    // grouped) and its GPU time added to its kernel kind; lapid_b200_take_profile drains the totals
    bool profile = false;
    std::map<std::string, std::pair<uint64_t, double>> profile_by_kind;
    std::vector<cudaEvent_t> profile_events;

    void make_current() const { cuda_check(cudaSetDevice(ordinal), "cudaSetDevice"); }
    ~lapid_b200_device() {
        if (cudaSetDevice(ordinal) == cudaSuccess) {
            if (scratch) cudaFree(scratch);
            if (stream_ws.pairs) cudaFree(stream_ws.pairs);
            if (status_host) cudaFreeHost(status_host);
            for (cudaEvent_t e : profile_events) cudaEventDestroy(e);
            for (cudaEvent_t e : io_events) cudaEventDestroy(e);
            if (io_in) cudaStreamDestroy(io_in);
            if (io_out) cudaStreamDestroy(io_out);
            if (own_stream) cudaStreamDestroy(own_stream);
        }
    }
    // Grow-only scratch; growing waits for the stream first (nothing may still use the old block).
    void ensure_scratch(size_t bytes) {
        if (bytes <= scratch_bytes) return;
        cuda_check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
        if (scratch) cuda_check(cudaFree(scratch), "cudaFree");
        scratch = nullptr;
        scratch_bytes = 0;
        size_t want = (bytes + (1u << 20) - 1) & ~(size_t)((1u << 20) - 1);
        cuda_check(cudaMalloc(&scratch, want), "cudaMalloc(scratch)");
        scratch_bytes = want;
    }
};

struct lapid_b200_buffer {
    std::atomic<int> refs{1};
    lapid_b200_device *dev = nullptr;  // retained
    void *ptr = nullptr;
    size_t bytes = 0;
    bool owned = true;
};

namespace {

void device_release(lapid_b200_device *d) {
    if (d && d->refs.fetch_sub(1) == 1) delete d;
}

void buffer_release(lapid_b200_buffer *b) {
    if (!b || b->refs.fetch_sub(1) != 1) return;
    if (b->owned && b->ptr && cudaSetDevice(b->dev->ordinal) == cudaSuccess) {
        // frees are ordered after the work queued on the device's stream
        cudaStreamSynchronize(b->dev->stream);
        cudaFree(b->ptr);
    }
    device_release(b->dev);
    delete b;
}

lapid_b200_device *need(lapid_b200_device *d) {
    if (!d) fail("invalid_argument", "device is NULL");
    return d;
}
lapid_b200_buffer *need(lapid_b200_buffer *b, const char *what) {
    if (!b) fail("invalid_argument", std::string(what) + " is NULL");
    return b;
}

lapid_b200_buffer *new_buffer(lapid_b200_device *dev, void *ptr, size_t bytes, bool owned) {
    auto *b = new lapid_b200_buffer();
    dev->refs.fetch_add(1);
    b->dev = dev;
    b->ptr = ptr;
    b->bytes = bytes;
    b->owned = owned;
    return b;
}

// ------------------------------------------------------------------ launch validation + dispatch
struct Plan {
    bool noop = false;
    bool zero_k = false;
    bool gemv = false;
    uint32_t rows = 0;
    lapid_b200_layout wl{};
    size_t scratch = 0;  // bytes of activation scratch the launch needs
    bool fast = false;   // specialised Q4_K / Q6_K GEMV (activations as 336-byte records)
    bool mma = false;    // Q4_K GEMV on the int8 tensor-core instruction (activations as tiles)
    bool stream = false; // ... through the balanced-stream kernel (Q4_K, Q5_K)
    int records() const { return mma ? 2 : fast ? 1 : 0; }  // ActQuantArgs::records
    bool fast_i8 = false;  // specialised Int8 / Int4 GEMV with bulk-copy rings (activations as planes)
    bool tc = false;     // tensor-core GEMM (needs a bf16 copy of the activations in the scratch)
};

// Where the quantized activations of a decode launch live in the scratch, and who makes them.
struct ActSlot {
    const void *ptr = nullptr;  // key: the A operand
    uint64_t off = 0, bs = 0, rs = 0;
    uint32_t rows = 0, m = 0, k = 0;
    int records = 0;
    int a_type = 0;        // element type of the operand (ACT_F32 / ACT_F16 / ACT_BF16)
    size_t offset = 0;     // into the device scratch
    bool hoisted = false;  // quantized by the batched pre-pass at the head of the call
    bool done = false;
    bool same(const ActSlot &o) const {
        return ptr == o.ptr && off == o.off && bs == o.bs && rs == o.rs && rows == o.rows && m == o.m && k == o.k &&
               records == o.records && a_type == o.a_type;
    }
};

// Decode launches of one list that wait to go out as one grouped kernel: same format, rows and k,
// and none of them reads or overwrites what another one writes, so running them side by side
// gives what running them in order gives.
// A decode launch whose epilogue expression its kernel did not evaluate (the kernels store the plain accumulator then):
// one more kernel applies it in place.
void finish_expr(lapid_b200_device &dev, const lb::GemvArgs &it) {
    if (!it.epi.n) return;
    cuda_check(lb::launch_epilogue_expr(it.epi, it.out, it.out_off, it.out_bs, it.out_rs, it.extra, it.ex_off, it.ex_s0, it.ex_s1, it.ex_s2,
                                        it.rows / it.m, it.m, it.n, dev.sm_count, dev.stream), "epilogue launch");
    dev.launches++;
}

struct PendingGroup {
    struct Range {
        const char *lo, *hi;
        bool hits(const Range &o) const { return lo < o.hi && o.lo < hi; }
    };
    int fmt = 0, mode = 0;  // kernel of the members: 1 = dp4a kernel, 2 = tensor-core kernel, 3 = balanced-stream tensor-core kernel
    lb::GemvGroup g{};
    bool split_early = false;  // see accepts()
    std::vector<Range> writes, reads;

    bool accepts(int f, int md, const lb::GemvArgs &a, const Range &out, const Range *in, int n_in) {
        if (g.count == 0) return true;
        if (g.count == lb::GEMV_GROUP_MAX || f != fmt || md != mode || a.rows != g.item[0].rows || a.k != g.item[0].k) return false;
        // In a long list, dp4a launches that may run ahead of their predecessor overlap on their own: measured (one row,
        // the three K = 4096 projections of an 8B layer inside a list of 16) 17.7 us as three launches against 19.2 us
        // as one. In a short list (q, k, v of one decoder layer) the launch boundaries weigh more: 80 layers of 70B
        // shapes take 9.8 ms per token grouped, 10.6 ms one by one.
        if (md == 1 && split_early && a.early && g.item[0].early) return false;
        for (const Range &w : writes) {
            if (w.hits(out)) return false;
            for (int i = 0; i < n_in; i++)
                if (w.hits(in[i])) return false;
        }
        for (const Range &r : reads)
            if (r.hits(out)) return false;
        g.item[g.count] = a;
        g.count++;
        bool fits = md == 3 ? true  // its shared memory does not depend on the members
                    : md != 2 ? lb::qgemv_kq_group_smem(f, g) <= 227 * 1024 - 256
                              : f == LAPID_B200_DTYPE_Q6_K ? lb::qgemv_q6k_mma_group_fits(g) : lb::qgemv_q4k_mma_group_fits(g);
        g.count--;
        return fits;
    }
    void add(int f, int md, const lb::GemvArgs &a, const Range &out, const Range *in, int n_in) {
        fmt = f;
        mode = md;
        g.item[g.count++] = a;
        writes.push_back(out);
        for (int i = 0; i < n_in; i++) reads.push_back(in[i]);
    }
    void flush(lapid_b200_device &dev) {
        if (g.count == 0) return;
        int count = g.count;
        g.count = 0;  // also when the launch fails: the list is abandoned then
        writes.clear();
        reads.clear();
        lb::GemvGroup out = g;
        out.count = count;
        const bool early = dev.early_ok(true);  // members carry early = 1 when their activations came from the pre-pass at the head
        for (int i = 0; i < count; i++) out.item[i].early = early ? out.item[i].early : 0;
        const bool pdl = dev.pdl_launch();
        const uint64_t before = dev.stream_ws.kernels;
        if (mode == 3) cuda_check(lb::launch_qgemv_kq_stream(fmt, out, dev.stream_ws, dev.sm_count, pdl, dev.stream), "qgemv launch");
        else if (mode == 2 && fmt == LAPID_B200_DTYPE_Q6_K) cuda_check(lb::launch_qgemv_q6k_mma(out, dev.sm_count, pdl, dev.stream), "qgemv launch");
        else if (mode == 2) cuda_check(lb::launch_qgemv_q4k_mma(out, dev.sm_count, pdl, dev.stream, dev.gemv_stream ? &dev.stream_ws : nullptr), "qgemv launch");
        else cuda_check(lb::launch_qgemv_kq_group(fmt, out, dev.sm_count, pdl, dev.stream), "qgemv launch");
        dev.launches += dev.stream_ws.kernels > before ? dev.stream_ws.kernels - before : 1;  // (the stream kernel may take two)
        for (int i = 0; i < count; i++) finish_expr(dev, out.item[i]);
    }
};

std::string dims_str(const lapid_b200_launch &l) {
    return "[" + std::to_string(l.batch) + ", " + std::to_string(l.m) + ", " + std::to_string(l.n) + ", " +
           std::to_string(l.k) + "]";
}

// The epilogue program of a launch: known nodes, a well-formed postfix order, at most four values on the stack, one
// result. Returns whether it loads extras[0].
bool check_expr(const lapid_b200_launch &l) {
    if (l.n_expr == 0 || l.n_expr > LAPID_B200_EXPR_WORDS)
        fail("invalid_launch", "b200 matmul: an epilogue expression of " + std::to_string(l.n_expr) + " words (1.." + std::to_string(LAPID_B200_EXPR_WORDS) + ")");
    int depth = 0;
    bool extra = false;
    for (uint32_t i = 0; i < l.n_expr; i++) {
        const uint32_t w = l.expr[i], op = w & 0xffu, arg = w >> 8;
        int pops = 0;
        if (op == LAPID_B200_EXPR_LOAD) {
            if (arg > 1) fail("unsupported", "b200 matmul: epilogue Load(" + std::to_string(arg) + "): one extra is supported");
            extra = extra || arg == 1;
        } else if (op == LAPID_B200_EXPR_CONST) {
            if (++i >= l.n_expr) fail("invalid_launch", "b200 matmul: epilogue expression ends inside a constant");
        } else if (op >= LAPID_B200_EXPR_NEG && op <= LAPID_B200_EXPR_ABS) {
            pops = 1;
        } else if (op >= LAPID_B200_EXPR_ADD && op <= LAPID_B200_EXPR_CMPEQ) {
            pops = 2;
        } else if (op == LAPID_B200_EXPR_WHERE) {
            pops = 3;
        } else {
            fail("unsupported", "b200 matmul: epilogue node " + std::to_string(op) + " (the f32 nodes of the expression type are supported)");
        }
        if (depth < pops) fail("invalid_launch", "b200 matmul: epilogue expression pops an empty stack at word " + std::to_string(i));
        depth += 1 - pops;
        if (depth > 4) fail("unsupported", "b200 matmul: epilogue expression needs more than four values on the stack");
    }
    if (depth != 1) fail("invalid_launch", "b200 matmul: epilogue expression leaves " + std::to_string(depth) + " values");
    return extra;
}

// Checks that need no buffers (prepare runs these alone).
Plan plan_launch(const lapid_b200_device &dev, const lapid_b200_launch &l) {
    Plan p;
    if (l.kind != LAPID_B200_KERNEL_MATMUL) fail("unsupported", "kernel kind " + std::to_string(l.kind) + " is not MatMul");
    if (!is_quant(l.b_dtype))
        fail("unsupported_dtype", "b200 matmul: b dtype " + std::to_string(l.b_dtype) + " (want int8, int4, q4_k, q5_k, q6_k, mxfp4 or an i-quant)");
    if ((!is_act_float(l.a_dtype) && l.a_dtype != LAPID_B200_DTYPE_ACT_Q8) || l.out_dtype != LAPID_B200_DTYPE_F32)
        fail("unsupported_dtype", "b200 matmul: a must be f32, f16 or bf16 and out f32");
    if (l.epilogue != LAPID_B200_EPILOGUE_NONE && l.epilogue != LAPID_B200_EPILOGUE_ADD && l.epilogue != LAPID_B200_EPILOGUE_EXPR)
        fail("unsupported", "b200 matmul: epilogue " + std::to_string(l.epilogue));
    const bool reads_extra = l.epilogue == LAPID_B200_EPILOGUE_ADD || (l.epilogue == LAPID_B200_EPILOGUE_EXPR && check_expr(l));
    int want_inputs = reads_extra ? 3 : 2;
    if (l.n_inputs != want_inputs)
        fail("invalid_launch", "expected " + std::to_string(want_inputs) + " inputs, got " + std::to_string(l.n_inputs));
    if (reads_extra && l.extra_dtype != LAPID_B200_DTYPE_F32) fail("unsupported_dtype", "b200 matmul: extra must be f32");
    const uint64_t lim = 1ull << 31;  // 32-bit indexing inside the kernels
    if (l.batch >= lim || l.m >= lim || l.n >= lim || l.k >= lim || l.batch * l.m >= lim)
        fail("too_large", "b200 matmul: dimensions " + dims_str(l) + " exceed 32-bit indexing");
    if (l.batch * l.m * l.n == 0) {
        p.noop = true;
        return p;
    }
    p.rows = (uint32_t)(l.batch * l.m);
    if (l.k == 0) {
        p.zero_k = true;
        return p;
    }
    if (!l.b_transposed || l.b.offset != 0 || l.b.batch_stride != 0)
        fail("invalid_launch", "b200 matmul: quantized B must be transposed with zero offset and batch stride");
    p.wl = layout_of(l.b_dtype, l.n, l.k);
    if (l.b.row_stride != l.k)
        fail("shape_mismatch", "b200 matmul: quantized B row stride " + std::to_string(l.b.row_stride) + ", expected k = " +
                                   std::to_string(l.k));
    p.gemv = p.rows <= dev.gemv_max_rows;
    if (l.a_dtype == LAPID_B200_DTYPE_ACT_Q8 && (!p.gemv || l.k % 256 != 0))
        fail("invalid_launch", "b200 matmul: a quantized activation operand needs batch*m <= " + std::to_string(dev.gemv_max_rows) +
                                   " and k a multiple of 256");
    if (p.gemv) {
        size_t qa = align_up((uint64_t)p.rows * l.k, 256);
        size_t sc = align_up((uint64_t)p.rows * (l.k / 32) * 4, 256);
        size_t rec = align_up((uint64_t)p.rows * ((l.k + 255) / 256) * lb::REC, 256);  // record layout of the fast path
        p.scratch = qa + 2 * sc > rec ? qa + 2 * sc : rec;
        p.fast = dev.gemv_fast && lb::qgemv_kq_fast_shape_ok(l.b_dtype, p.rows, (uint32_t)l.k);
        p.fast_i8 = dev.gemv_fast && (l.b_dtype == LAPID_B200_DTYPE_INT8 || l.b_dtype == LAPID_B200_DTYPE_INT4) &&
                    lb::qgemv_i8_fast_shape_ok(p.rows, (uint32_t)l.k);  // (Int4: the same kernel over nibble planes)
        // (Q6_K pays more per weight for unpacking: its tensor-core kernel wins one row later than Q4_K's)
        p.stream = dev.gemv_fast && dev.gemv_mma_rows > 0 &&
                   ((dev.gemv_stream >= 2 && l.b_dtype == LAPID_B200_DTYPE_Q4_K && p.rows >= dev.gemv_mma_rows) ||
                    (dev.gemv_stream >= 1 && l.b_dtype == LAPID_B200_DTYPE_Q5_K && p.rows > dev.gemv_mma_rows)) &&
                   lb::qgemv_kq_stream_shape_ok(l.b_dtype, p.rows, (uint32_t)l.n, (uint32_t)l.k);
        p.mma = dev.gemv_fast && dev.gemv_mma_rows > 0 &&
                (p.stream ||
                 (l.b_dtype == LAPID_B200_DTYPE_Q4_K && p.rows >= dev.gemv_mma_rows && lb::qgemv_q4k_mma_shape_ok(p.rows, (uint32_t)l.k)) ||
                 (l.b_dtype == LAPID_B200_DTYPE_Q6_K && p.rows > dev.gemv_mma_rows && lb::qgemv_q6k_mma_shape_ok(p.rows, (uint32_t)l.k)) ||
                 (l.b_dtype == LAPID_B200_DTYPE_INT8 && p.rows >= dev.gemv_mma_rows && lb::qgemv_i8_mma_shape_ok(p.rows, (uint32_t)l.k)) ||
                 (l.b_dtype == LAPID_B200_DTYPE_INT4 && p.rows >= dev.gemv_mma_rows && lb::qgemv_i4_mma_shape_ok(p.rows, (uint32_t)l.k)) ||
                 (l.b_dtype == LAPID_B200_DTYPE_MXFP4 && dev.mxfp4_mma_rows > 0 && p.rows >= dev.mxfp4_mma_rows &&
                  lb::qgemv_mxfp4_mma_shape_ok(p.rows, (uint32_t)l.k)));
        // Small Q5_K / Q6_K matrices at three and four rows: their tensor-core kernels cost about 5 us whatever the size
        // (1024 x 4096: 5.0-5.5 us), the dp4a kernel 3.8-4.6 us; from five rows on, and from 4096 x 4096 on, the
        // tensor-core kernels win.
        if (p.fast && p.rows <= 4 && (uint64_t)l.n * l.k <= (6ull << 20) &&
            (l.b_dtype == LAPID_B200_DTYPE_Q5_K || l.b_dtype == LAPID_B200_DTYPE_Q6_K) && dev.small_dp4a) {
            p.stream = false;
            p.mma = false;
        }
        if (p.mma) {
            size_t tiles = align_up(lb::qgemv_q4k_mma_act_bytes(p.rows, (uint32_t)l.k), 256);
            if (tiles > p.scratch) p.scratch = tiles;
        }
    } else {
        p.tc = !dev.gemm_f32 && l.k % 256 == 0 && l.k >= 256 &&
               (l.b_dtype == LAPID_B200_DTYPE_Q4_K || l.b_dtype == LAPID_B200_DTYPE_Q5_K || l.b_dtype == LAPID_B200_DTYPE_Q6_K);
        if (p.tc) p.scratch = align_up(lb::qgemm_tc_scratch_bytes(p.rows, (uint32_t)l.n, (uint32_t)l.k, dev.sm_count), 256);
    }
    return p;
}

// The quantized activation operand of a decode launch inside `base`: planes, records or tiles.
lb::ActOut act_out_at(void *base, int records, uint32_t rows, uint32_t k) {
    lb::ActOut o{};
    o.qa = (int8_t *)base;
    o.da = (float *)((char *)base + lb::act_plane_bytes(rows, k));
    o.bs = (float *)((char *)base + lb::act_plane_bytes(rows, k) + lb::act_scale_bytes(rows, k));
    o.records = records;
    o.rows = rows;
    o.k = k;
    return o;
}

// What the `_act` producers need to know about the buffer they fill.
lb::ActOut act_out_checked(lapid_b200_device *dev, lapid_b200_buffer *qact, int32_t layout, uint64_t rows, uint64_t cols, const char *who) {
    lb::ActOut o{};
    if (!qact) return o;
    if (qact->dev != dev) fail("wrong_backend", std::string(who) + ": qact belongs to another device");
    if (layout < 0 || layout > 2) fail("invalid_argument", std::string(who) + ": layout must be 0, 1 or 2");
    if (rows == 0 || rows > 8 || cols % 256 != 0 || cols == 0 || cols >= (1ull << 31))
        fail("invalid_launch", std::string(who) + ": a quantized copy needs rows in 1..8 and cols a multiple of 256");
    const size_t planes = lb::act_plane_bytes((uint32_t)rows, (uint32_t)cols) + 2 * lb::act_scale_bytes((uint32_t)rows, (uint32_t)cols);
    const size_t need_b = layout == 0 ? planes : layout == 1 ? rows * (cols / 256) * lb::REC : lb::qgemv_q4k_mma_act_bytes((uint32_t)rows, (uint32_t)cols);
    if (qact->bytes < need_b) fail("out_of_bounds", std::string(who) + " qact: needs " + std::to_string(need_b) + " bytes, buffer has " + std::to_string(qact->bytes));
    if ((uintptr_t)qact->ptr & 15) fail("invalid_launch", std::string(who) + ": qact must be 16-byte aligned");
    return act_out_at(qact->ptr, layout, (uint32_t)rows, (uint32_t)cols);
}

// `tp` not null: a launch that takes one of the K-quant fast decode kernels hands its result to the
// tensor-parallel group from its epilogue instead of storing it (`*pushed` says whether it did).
// Kernel::Gather: out[i, :] = dequant(table[ids[i], :]).
void check_gather(const lapid_b200_launch &l) {
    const bool quant = is_quant(l.b_dtype);
    if (!quant && l.b_dtype != LAPID_B200_DTYPE_F32)
        fail("unsupported_dtype", "b200 gather: table dtype " + std::to_string(l.b_dtype) + " (want f32, int8, int4, q4_k, q5_k, q6_k, mxfp4 or an i-quant)");
    if (l.out_dtype != LAPID_B200_DTYPE_F32) fail("unsupported_dtype", "b200 gather: out must be f32");
    if (l.n_inputs != 2) fail("invalid_launch", "expected 2 inputs, got " + std::to_string(l.n_inputs));
    if (l.batch != 1) fail("invalid_launch", "b200 gather: batch must be 1");
    const uint64_t lim = 1ull << 31;
    if (l.m >= lim || l.n >= lim || l.k >= lim) fail("too_large", "b200 gather: dimensions exceed 32-bit indexing");
}

void run_gather(lapid_b200_device &dev, const lapid_b200_launch &l, lapid_b200_buffer *const *buffers, size_t n_buffers) {
    check_gather(l);
    auto get = [&](uint32_t id) -> lapid_b200_buffer * {
        if (id >= n_buffers || !buffers[id])
            fail("invalid_launch", "buffer id " + std::to_string(id) + " out of range (" + std::to_string(n_buffers) + " buffers)");
        if (buffers[id]->dev != &dev) fail("wrong_backend", "buffer " + std::to_string(id) + " belongs to another device");
        return buffers[id];
    };
    lapid_b200_buffer *out = get(l.output), *table = get(l.inputs[0]), *ids = get(l.inputs[1]);
    if (table->ptr == out->ptr || ids->ptr == out->ptr) fail("buffer_aliasing", "gather: an input buffer is the output buffer");
    const uint64_t rows = l.k, cols = l.n, count = l.m;
    if (count == 0 || cols == 0) return;
    if (ids->bytes / 4 < count) fail("out_of_bounds", "gather indices: need " + std::to_string(count) + " i32, buffer holds " + std::to_string(ids->bytes / 4));
    if (out->bytes / 4 < count * cols)
        fail("out_of_bounds", "gather output: need " + std::to_string(count * cols) + " f32, buffer holds " + std::to_string(out->bytes / 4));
    uint64_t scales_offset = 0;
    int fmt = -1;
    if (is_quant(l.b_dtype)) {
        lapid_b200_layout wl = layout_of(l.b_dtype, rows, cols);
        if (table->bytes < wl.scales_offset + wl.scales_bytes)
            fail("out_of_bounds", "gather: quantized [" + std::to_string(rows) + ", " + std::to_string(cols) + "] needs " +
                                      std::to_string(wl.total) + " bytes, buffer has " + std::to_string(table->bytes));
        scales_offset = wl.scales_offset;
        fmt = l.b_dtype;
    } else if (table->bytes / 4 < rows * cols) {
        fail("out_of_bounds", "gather table: need " + std::to_string(rows * cols) + " f32, buffer holds " + std::to_string(table->bytes / 4));
    }
    cuda_check(lb::launch_gather(fmt, table->ptr, scales_offset, (const int32_t *)ids->ptr, rows, cols, count, (float *)out->ptr,
                                 dev.status_dev, dev.sm_count, dev.stream), "gather launch");
    dev.launches++;
}

// Kernel::MatMulId (ir.rs:425-443): out[t, s, :] = W[ids[t, s]] x[t]. In the launch: m = t, batch = r (slots per
// token), b.batch_stride = e (matrices in the stack), n, k; inputs = {x, w, ids}.
struct MoePlan {
    bool noop = false, zero_k = false;
    bool decode = false;  // t <= gemv_max_rows: int8-activation arithmetic, one one-row GEMV per pair
    bool fast = false;    // decode: the K-quant kernel with bulk-copy rings (activations as records)
    bool tc = false;      // above decode sizes: tensor cores (else the exact f32 kernel)
    uint32_t mt = 64;     // activation rows per tile of the grouped GEMM
    uint64_t t = 0, r = 0, e = 0;
    lapid_b200_layout wl{};
    size_t route_bytes = 0, scratch = 0;
};

MoePlan plan_matmul_id(const lapid_b200_device &dev, const lapid_b200_launch &l) {
    MoePlan p;
    if (!is_quant(l.b_dtype))
        fail("unsupported_dtype", "b200 matmul_id: w dtype " + std::to_string(l.b_dtype) + " (want int8, int4, q4_k, q5_k, q6_k, mxfp4 or an i-quant)");
    if (l.a_dtype != LAPID_B200_DTYPE_F32 || l.out_dtype != LAPID_B200_DTYPE_F32)
        fail("unsupported_dtype", "b200 matmul_id: x and out must be f32");
    if (l.epilogue != LAPID_B200_EPILOGUE_NONE) fail("unsupported", "b200 matmul_id: no epilogue");
    if (l.n_inputs != 3) fail("invalid_launch", "expected 3 inputs (x, w, ids), got " + std::to_string(l.n_inputs));
    p.t = l.m;
    p.r = l.batch;
    p.e = l.b.batch_stride;
    const uint64_t lim = 1ull << 31;
    if (p.t >= lim || p.r >= lim || p.e >= lim || l.n >= lim || l.k >= lim || p.t * p.r >= lim || p.t * p.r * l.n >= (1ull << 40))
        fail("too_large", "b200 matmul_id: dimensions exceed 32-bit indexing");
    if (p.t * p.r * l.n == 0) {
        p.noop = true;
        return p;
    }
    if (l.k == 0) {
        p.zero_k = true;
        return p;
    }
    p.wl = layout_of(l.b_dtype, l.n, l.k);
    p.decode = p.t <= dev.gemv_max_rows;
    if (p.decode) {
        if (p.t * p.r > 65535) fail("too_large", "b200 matmul_id: more than 65535 (token, slot) pairs in a decode-sized launch");
        p.fast = dev.gemv_fast && lb::qgemv_kq_moe_shape_ok(l.b_dtype, (uint32_t)p.t, (uint32_t)l.k);
        size_t qa = align_up(p.t * l.k, 256), sc = align_up(p.t * (l.k / 32) * 4, 256);
        size_t rec = align_up(p.t * ((l.k + 255) / 256) * lb::REC, 256);
        p.scratch = p.fast ? rec : qa + 2 * sc;
    } else {
        p.tc = !dev.gemm_f32 && lb::qgemm_tc_moe_supported(l.b_dtype, p.e, l.n, l.k, nullptr);
        if (p.tc) {
            const uint64_t avg = p.t * p.r / (p.e ? p.e : 1);
            // the grouped GEMM is bound by dequantization, which is paid once per (weight tile, activation tile):
            // prefer the tile that holds an expert's expected rows (plus the spread of a random routing) in one piece
            p.mt = avg <= 48 ? 64 : avg <= 100 ? 128 : 256;
        }
        if ((uint64_t)lb::moe_max_tiles(p.t * p.r, p.e, p.mt) * p.mt >= lim) fail("too_large", "b200 matmul_id: tile space exceeds 32-bit indexing");
        p.route_bytes = lb::moe_route_bytes(p.t * p.r, p.e, p.mt);
        p.scratch = p.route_bytes;
        if (p.tc) p.scratch += align_up((uint64_t)lb::moe_max_tiles(p.t * p.r, p.e, p.mt) * p.mt * l.k * 2, 256);
    }
    return p;
}

void run_matmul_id(lapid_b200_device &dev, const lapid_b200_launch &l, lapid_b200_buffer *const *buffers, size_t n_buffers,
                   const ActSlot *slot) {
    MoePlan p = plan_matmul_id(dev, l);
    auto get = [&](uint32_t id) -> lapid_b200_buffer * {
        if (id >= n_buffers || !buffers[id])
            fail("invalid_launch", "buffer id " + std::to_string(id) + " out of range (" + std::to_string(n_buffers) + " buffers)");
        if (buffers[id]->dev != &dev) fail("wrong_backend", "buffer " + std::to_string(id) + " belongs to another device");
        return buffers[id];
    };
    lapid_b200_buffer *out = get(l.output), *x = get(l.inputs[0]), *w = get(l.inputs[1]), *ids = get(l.inputs[2]);
    if (x->ptr == out->ptr || w->ptr == out->ptr || ids->ptr == out->ptr)
        fail("buffer_aliasing", "matmul_id: an input buffer is the output buffer");
    if (p.noop) return;
    const uint64_t pairs = p.t * p.r;
    if (ids->bytes / 4 < pairs || x->bytes / 4 < p.t * l.k || out->bytes / 4 < pairs * l.n)
        fail("out_of_bounds", "b200 matmul_id: buffers too small for t=" + std::to_string(p.t) + " r=" + std::to_string(p.r) +
                                  " n=" + std::to_string(l.n) + " k=" + std::to_string(l.k));
    if (p.zero_k) {
        cuda_check(cudaMemsetAsync(out->ptr, 0, pairs * l.n * 4, dev.stream), "memset");
        return;
    }
    if (p.e == 0) fail("invalid_launch", "b200 matmul_id: the expert stack is empty");
    if (w->bytes < p.e * p.wl.total)
        fail("out_of_bounds", "b200 matmul_id: expert stack holds " + std::to_string(w->bytes) + " < " + std::to_string(p.e * p.wl.total) + " bytes");
    if (((uintptr_t)w->ptr & 15) != 0 || ((uintptr_t)x->ptr & 15) != 0) fail("invalid_launch", "b200 matmul_id: x and w must be 16-byte aligned");
    size_t off = 0;
    if (slot) off = slot->offset;
    else dev.ensure_scratch(p.scratch);
    char *base = (char *)dev.scratch + off;
    if (p.decode) {
        size_t qa_b = align_up(p.t * l.k, 256), sc_b = align_up(p.t * (l.k / 32) * 4, 256);
        lb::ActQuantArgs q{};
        q.a = (const float *)x->ptr;
        q.a_rs = l.k;
        q.rows = (uint32_t)p.t;
        q.m = (uint32_t)p.t;
        q.k = (uint32_t)l.k;
        q.qa = (int8_t *)base;
        q.da = (float *)(base + qa_b);
        q.bs = has_min_term(l.b_dtype) ? (float *)(base + qa_b + sc_b) : nullptr;
        q.records = p.fast ? 1 : 0;
        cuda_check(lb::launch_act_quant(q, dev.sm_count, dev.pdl_launch(), dev.stream), "act_quant launch");
        lb::GemvArgs g{};
        g.w = (const uint8_t *)w->ptr;
        g.w_bytes = w->bytes;
        g.scales_offset = p.wl.scales_offset;
        g.qa = q.qa;
        g.da = q.da;
        g.bs = q.bs;
        g.status = dev.status_dev;
        g.out = (float *)out->ptr;
        g.out_rs = l.n;
        g.rows = (uint32_t)p.t;
        g.m = (uint32_t)p.t;
        g.n = (uint32_t)l.n;
        g.k = (uint32_t)l.k;
        g.ids = (const int32_t *)ids->ptr;
        g.id_stride = p.wl.total;
        g.id_r = (uint32_t)p.r;
        g.id_e = (uint32_t)p.e;
        const bool pdl = dev.pdl_launch();
        if (l.b_dtype == LAPID_B200_DTYPE_INT4) cuda_check(lb::launch_qgemv_i4(g, dev.sm_count, pdl, dev.stream), "matmul_id launch");
        else if (l.b_dtype == LAPID_B200_DTYPE_MXFP4) cuda_check(lb::launch_qgemv_mxfp4(g, dev.sm_count, pdl, dev.stream), "matmul_id launch");
        else if (is_iquant(l.b_dtype)) cuda_check(lb::launch_qgemv_iq(l.b_dtype, g, dev.sm_count, pdl, dev.stream), "matmul_id launch");
        else if (p.fast) cuda_check(lb::launch_qgemv_kq_moe(l.b_dtype, g, dev.sm_count, pdl, dev.stream), "matmul_id launch");
        else cuda_check(lb::launch_qgemv_moe(l.b_dtype, g, dev.sm_count, pdl, dev.stream), "matmul_id launch");
        dev.launches += 2;
        return;
    }
    lb::MoeRouteArgs route{};
    lb::moe_route_layout(base, pairs, p.e, p.mt, route);
    route.ids = (const int32_t *)ids->ptr;
    route.status = dev.status_dev;
    cuda_check(lb::launch_moe_route(route, dev.pdl_launch(), dev.stream), "matmul_id route launch");
    dev.launches++;
    const uint32_t rows = route.max_tiles * route.mt;
    if (p.tc && lb::qgemm_tc_moe_supported(l.b_dtype, p.e, l.n, l.k, w->ptr) && p.wl.total == p.wl.qs_bytes) {
        void *a_bf16 = base + p.route_bytes;
        cuda_check(lb::launch_moe_gather_bf16((const float *)x->ptr, route, (uint32_t)p.r, (uint32_t)l.k, a_bf16, dev.stream), "matmul_id gather launch");
        lb::GemmTcArgs t{};
        t.w = (const uint8_t *)w->ptr;
        t.out = (float *)out->ptr;
        t.rows = rows;
        t.m = rows;
        t.n = (uint32_t)l.n;
        t.k = (uint32_t)l.k;
        t.status = dev.status_dev;
        t.tile_expert = route.tile_expert;
        t.row_pair = route.row_pair;
        cuda_check(lb::launch_qgemm_tc_moe(l.b_dtype, t, (uint32_t)p.e, p.mt, a_bf16, dev.stream), "matmul_id gemm launch");
        dev.launches += 2;
        return;
    }
    lb::GemmF32Args f{};
    f.w = (const uint8_t *)w->ptr;
    f.scales_offset = p.wl.scales_offset;
    f.a = (const float *)x->ptr;
    f.a_rs = l.k;
    f.out = (float *)out->ptr;
    f.rows = rows;
    f.m = rows;
    f.n = (uint32_t)l.n;
    f.k = (uint32_t)l.k;
    f.tile_expert = route.tile_expert;
    f.row_pair = route.row_pair;
    f.id_stride = p.wl.total;
    f.id_r = (uint32_t)p.r;
    cuda_check(lb::launch_qgemm_f32(l.b_dtype, f, dev.stream), "matmul_id gemm launch");
    dev.launches++;
}

void run_launch(lapid_b200_device &dev, const lapid_b200_launch &l, lapid_b200_buffer *const *buffers, size_t n_buffers,
                ActSlot *slot, PendingGroup *pend = nullptr, const lb::TpPushTable *tp = nullptr, bool *pushed = nullptr) {
    if (l.kind == LAPID_B200_KERNEL_GATHER) {
        if (pend) pend->flush(dev);
        run_gather(dev, l, buffers, n_buffers);
        return;
    }
    if (l.kind == LAPID_B200_KERNEL_MATMUL_ID) {
        if (pend) pend->flush(dev);
        run_matmul_id(dev, l, buffers, n_buffers, slot);
        return;
    }
    Plan p = plan_launch(dev, l);
    auto get = [&](uint32_t id) -> lapid_b200_buffer * {
        if (id >= n_buffers || !buffers[id])
            fail("invalid_launch", "buffer id " + std::to_string(id) + " out of range (" + std::to_string(n_buffers) + " buffers)");
        if (buffers[id]->dev != &dev) fail("wrong_backend", "buffer " + std::to_string(id) + " belongs to another device");
        return buffers[id];
    };
    lapid_b200_buffer *out = get(l.output);
    lapid_b200_buffer *ins[3] = {nullptr, nullptr, nullptr};
    for (int i = 0; i < l.n_inputs; i++) {
        ins[i] = get(l.inputs[i]);
        if (ins[i]->ptr == out->ptr)
            fail("buffer_aliasing", "input buffer " + std::to_string(l.inputs[i]) + " is the output buffer " + std::to_string(l.output));
    }
    if (p.noop) return;
    uint64_t out_elems = out->bytes / 4;
    uint64_t last = l.out.offset + (l.batch - 1) * l.out.batch_stride + (l.m - 1) * l.out.row_stride + l.n;
    if (out_elems < last)
        fail("out_of_bounds", "b200 matmul: output holds " + std::to_string(out_elems) + " < " + std::to_string(last) + " elements");
    if (l.k > 0 && l.a_dtype != LAPID_B200_DTYPE_ACT_Q8) {
        uint64_t alast = l.a.offset + (l.batch - 1) * l.a.batch_stride + (l.m - 1) * l.a.row_stride + l.k;
        if (ins[0]->bytes / act_elem_size(l.a_dtype) < alast)
            fail("out_of_bounds", "b200 matmul a: view reaches element " + std::to_string(alast) + ", buffer holds " +
                                      std::to_string(ins[0]->bytes / act_elem_size(l.a_dtype)));
    }
    const float *extra = nullptr;
    if (l.n_inputs == 3) {  // (plan_launch has matched the count to what the epilogue reads)
        // lowest and highest element the view touches over [batch, m, n]
        int64_t lo = (int64_t)l.extra.offset, hi = (int64_t)l.extra.offset;
        const uint64_t ext[3] = {l.batch, l.m, l.n};
        for (int d = 0; d < 3; d++) {
            int64_t span = l.extra.strides[d] * (int64_t)(ext[d] - 1);
            (span < 0 ? lo : hi) += span;
        }
        if (lo < 0 || (uint64_t)hi >= ins[2]->bytes / 4)
            fail("out_of_bounds", "b200 matmul extra 0: view spans [" + std::to_string(lo) + ", " + std::to_string(hi) +
                                      "], buffer holds " + std::to_string(ins[2]->bytes / 4));
        extra = (const float *)ins[2]->ptr;
    }

    lb::GemvArgs g{};
    g.out = (float *)out->ptr;
    g.out_off = l.out.offset;
    g.out_bs = l.out.batch_stride;
    g.out_rs = l.out.row_stride;
    g.extra = extra;
    g.ex_off = l.extra.offset;
    g.ex_s0 = l.extra.strides[0];
    g.ex_s1 = l.extra.strides[1];
    g.ex_s2 = l.extra.strides[2];
    if (l.epilogue == LAPID_B200_EPILOGUE_EXPR) {
        g.epi.n = l.n_expr;
        for (uint32_t i = 0; i < l.n_expr; i++) g.epi.code[i] = l.expr[i];
        if (tp) fail("unsupported", "b200: a row-parallel launch adds partial sums up; an epilogue expression cannot be applied to them");
    }
    g.rows = p.rows;
    g.m = (uint32_t)l.m;
    g.n = (uint32_t)l.n;
    g.k = (uint32_t)l.k;
    if (pend && !(p.gemv && !p.zero_k)) pend->flush(dev);  // anything but a decode launch ends the group
    // a prefill launch (and the k == 0 fill) with an expression stores plain results first; one more kernel applies it
    auto expr_pass = [&]() {
        if (!g.epi.n) return;
        cuda_check(lb::launch_epilogue_expr(g.epi, g.out, g.out_off, g.out_bs, g.out_rs, extra, g.ex_off, g.ex_s0, g.ex_s1, g.ex_s2,
                                            (uint32_t)l.batch, g.m, g.n, dev.sm_count, dev.stream), "epilogue launch");
        dev.launches++;
    };
    if (p.zero_k) {
        lb::GemvArgs z = g;
        if (g.epi.n) z.extra = nullptr;
        cuda_check(lb::launch_fill_zero_k(z, dev.stream), "fill launch");
        dev.launches++;
        expr_pass();
        return;
    }
    {   // the blocks themselves, to the end of their last 16-byte line (the Q6_K bulk copies fetch whole lines: 210-byte
        // blocks end anywhere); `layout().total`, which quantize hands out, is padded further
        const uint64_t need = align_up(p.wl.scales_offset + p.wl.scales_bytes, 16);
        if (ins[1]->bytes < need)
            fail("out_of_bounds", "b200: quantized [" + std::to_string(l.n) + ", " + std::to_string(l.k) + "] needs " + std::to_string(need) +
                                      " bytes (layout total " + std::to_string(p.wl.total) + "), buffer has " + std::to_string(ins[1]->bytes));
    }
    if (((uintptr_t)ins[1]->ptr & 15) != 0) fail("invalid_launch", "b200: quantized B must be 16-byte aligned");

    if (p.gemv) {
        ActSlot local;
        char *base = nullptr;
        if (l.a_dtype == LAPID_B200_DTYPE_ACT_Q8) {  // quantized by its producer (the `_act` glue kernels): no pre-pass
            if (ins[0]->bytes < p.scratch)
                fail("out_of_bounds", "b200 matmul: quantized activation operand needs " + std::to_string(p.scratch) + " bytes, buffer has " +
                                          std::to_string(ins[0]->bytes));
            if ((uintptr_t)ins[0]->ptr & 15) fail("invalid_launch", "b200 matmul: quantized activation operand must be 16-byte aligned");
            local.records = p.records();
            local.done = true;
            local.hoisted = true;  // complete before the list began (see execute_impl)
            slot = &local;
            base = (char *)ins[0]->ptr;
        } else {
            if (!slot) {  // not planned by the caller: a private slot at the start of the scratch
                dev.ensure_scratch(p.scratch);
                local.records = p.records();
                slot = &local;
            }
            base = (char *)dev.scratch + slot->offset;
        }
        size_t qa_b = align_up((uint64_t)p.rows * l.k, 256), sc_b = align_up((uint64_t)p.rows * (l.k / 32) * 4, 256);
        lb::ActQuantArgs q{};
        q.a = ins[0]->ptr;
        q.a_type = act_type_of(l.a_dtype);
        q.a_off = l.a.offset;
        q.a_bs = l.a.batch_stride;
        q.a_rs = l.a.row_stride;
        q.rows = p.rows;
        q.m = (uint32_t)l.m;
        q.k = (uint32_t)l.k;
        q.qa = (int8_t *)base;
        q.da = (float *)(base + qa_b);
        q.bs = (float *)(base + qa_b + sc_b);  // written for every format (a later launch may share the slot); read by Q4_K / Q5_K
        q.records = slot->records;
        g.w = (const uint8_t *)ins[1]->ptr;
        g.w_bytes = ins[1]->bytes;
        g.scales_offset = p.wl.scales_offset;
        g.qa = q.qa;
        g.da = q.da;
        g.bs = has_min_term(l.b_dtype) ? q.bs : nullptr;
        g.a = l.a_dtype == LAPID_B200_DTYPE_F32 ? (const float *)q.a : nullptr;
        g.a_off = q.a_off;
        g.a_bs = q.a_bs;
        g.a_rs = q.a_rs;
        g.status = dev.status_dev;
        if (pend && slot->records && l.b_dtype != LAPID_B200_DTYPE_INT8 && l.b_dtype != LAPID_B200_DTYPE_INT4 &&
            l.b_dtype != LAPID_B200_DTYPE_MXFP4) {  // (the Int8 / Int4 / MXFP4 kernels take one launch at a time)
            using Range = PendingGroup::Range;
            const char *ob = (const char *)out->ptr;
            Range wr{ob + 4 * l.out.offset, ob + 4 * last};
            Range in[3];
            int n_in = 0;
            for (int i = 0; i < l.n_inputs; i++) in[n_in++] = Range{(const char *)ins[i]->ptr, (const char *)ins[i]->ptr + ins[i]->bytes};
            const int mode = slot->records == 2 && p.stream ? 3 : slot->records;
            g.early = slot->hoisted ? 1 : 0;  // gated again when the group goes out
            if (!pend->accepts(l.b_dtype, mode, g, wr, in, n_in)) pend->flush(dev);
            if (!slot->done) {  // its input is not written by a pending launch (checked above), so it may run first
                cuda_check(lb::launch_act_quant(q, dev.sm_count, dev.pdl_launch(), dev.stream), "act_quant launch");
                dev.launches++;
                slot->done = true;
            }
            pend->add(l.b_dtype, mode, g, wr, in, n_in);
            return;
        }
        if (pend) pend->flush(dev);
        if (!slot->done) {
            cuda_check(lb::launch_act_quant(q, dev.sm_count, dev.pdl_launch(), dev.stream), "act_quant launch");
            dev.launches++;
            slot->done = true;
        }
        if (tp && slot->records) {
            g.tp = tp;
            *pushed = true;
        }
        g.early = dev.early_ok(slot->hoisted) ? 1 : 0;
        const bool pdl = dev.pdl_launch();
        const uint64_t ws_before = dev.stream_ws.kernels;
        if (slot->records == 2 && l.b_dtype == LAPID_B200_DTYPE_MXFP4) {
            cuda_check(lb::launch_qgemv_mxfp4_mma(g, dev.sm_count, pdl, dev.stream), "qgemv launch");
        } else if (slot->records == 2 && l.b_dtype == LAPID_B200_DTYPE_INT4) {
            cuda_check(lb::launch_qgemv_i4_mma(g, dev.sm_count, pdl, dev.stream), "qgemv launch");
        } else if (slot->records == 2 && l.b_dtype == LAPID_B200_DTYPE_INT8) {
            cuda_check(lb::launch_qgemv_i8_mma(g, dev.sm_count, pdl, dev.stream), "qgemv launch");
        } else if (slot->records == 2) {
            lb::GemvGroup one{};
            one.count = 1;
            one.item[0] = g;
            if (p.stream) cuda_check(lb::launch_qgemv_kq_stream(l.b_dtype, one, dev.stream_ws, dev.sm_count, pdl, dev.stream), "qgemv launch");
            else if (l.b_dtype == LAPID_B200_DTYPE_Q6_K) cuda_check(lb::launch_qgemv_q6k_mma(one, dev.sm_count, pdl, dev.stream), "qgemv launch");
            else cuda_check(lb::launch_qgemv_q4k_mma(one, dev.sm_count, pdl, dev.stream, dev.gemv_stream ? &dev.stream_ws : nullptr), "qgemv launch");
            g.epi.n = one.item[0].epi.n;  // (cleared when the launch evaluated its expression itself)
        } else if (slot->records) cuda_check(lb::launch_qgemv_kq_fast(l.b_dtype, g, dev.sm_count, pdl, dev.stream), "qgemv launch");
        else if (l.b_dtype == LAPID_B200_DTYPE_INT4 && p.fast_i8 && ((uintptr_t)g.w & 15) == 0 && (g.scales_offset & 15) == 0)
            cuda_check(lb::launch_qgemv_i4_fast(g, dev.sm_count, pdl, dev.stream), "qgemv launch");
        else if (l.b_dtype == LAPID_B200_DTYPE_INT4) cuda_check(lb::launch_qgemv_i4(g, dev.sm_count, pdl, dev.stream), "qgemv launch");
        else if (l.b_dtype == LAPID_B200_DTYPE_MXFP4) cuda_check(lb::launch_qgemv_mxfp4(g, dev.sm_count, pdl, dev.stream), "qgemv launch");
        else if (is_iquant(l.b_dtype)) cuda_check(lb::launch_qgemv_iq(l.b_dtype, g, dev.sm_count, pdl, dev.stream), "qgemv launch");
        else if (p.fast_i8 && ((uintptr_t)g.w & 15) == 0) cuda_check(lb::launch_qgemv_i8_fast(g, dev.sm_count, pdl, dev.stream), "qgemv launch");
        else cuda_check(lb::launch_qgemv(l.b_dtype, g, dev.sm_count, pdl, dev.stream), "qgemv launch");
        dev.launches += dev.stream_ws.kernels > ws_before ? dev.stream_ws.kernels - ws_before : 1;  // (the stream kernel may take two)
        finish_expr(dev, g);
        return;
    }
    if (p.tc) {
        lb::GemmTcArgs t{};
        t.w = (const uint8_t *)ins[1]->ptr;
        t.a = ins[0]->ptr;
        t.a_type = act_type_of(l.a_dtype);
        t.a_off = l.a.offset;
        t.a_bs = l.a.batch_stride;
        t.a_rs = l.a.row_stride;
        t.out = g.out;
        t.out_off = g.out_off;
        t.out_bs = g.out_bs;
        t.out_rs = g.out_rs;
        t.extra = g.epi.n ? nullptr : extra;
        t.ex_off = g.ex_off;
        t.ex_s0 = g.ex_s0;
        t.ex_s1 = g.ex_s1;
        t.ex_s2 = g.ex_s2;
        t.rows = p.rows;
        t.m = g.m;
        t.n = g.n;
        t.k = g.k;
        t.status = dev.status_dev;
        if (lb::qgemm_tc_supported(l.b_dtype, t)) {
            size_t off = 0;
            if (slot) off = slot->offset;
            else dev.ensure_scratch(p.scratch);
            int launched = 0;
            cuda_check(lb::launch_qgemm_tc(l.b_dtype, t, (char *)dev.scratch + off, dev.sm_count, dev.stream, &launched), "qgemm_tc launch");
            dev.launches += launched;
            expr_pass();
            return;
        }
    }
    lb::GemmF32Args f{};
    f.w = (const uint8_t *)ins[1]->ptr;
    f.scales_offset = p.wl.scales_offset;
    f.a = ins[0]->ptr;
    f.a_type = act_type_of(l.a_dtype);
    f.a_off = l.a.offset;
    f.a_bs = l.a.batch_stride;
    f.a_rs = l.a.row_stride;
    f.out = g.out;
    f.out_off = g.out_off;
    f.out_bs = g.out_bs;
    f.out_rs = g.out_rs;
    f.extra = g.epi.n ? nullptr : extra;
    f.ex_off = g.ex_off;
    f.ex_s0 = g.ex_s0;
    f.ex_s1 = g.ex_s1;
    f.ex_s2 = g.ex_s2;
    f.rows = p.rows;
    f.m = g.m;
    f.n = g.n;
    f.k = g.k;
    cuda_check(lb::launch_qgemm_f32(l.b_dtype, f, dev.stream), "qgemm_f32 launch");
    dev.launches++;
    expr_pass();
}

// After a wait on the device's stream: a kernel whose bounded wait gave up (or that met a bad index) said so in the
// host-visible status word; the call that notices fails, clears the word and leaves the device usable.
void check_status_word(lapid_b200_device *dev) {
    if (*dev->status_host == 0) return;
    int st = *dev->status_host;
    *dev->status_host = 0;
    // a launch that gave up may have left partial sums in the decode workspace
    cudaMemsetAsync(dev->stream_ws.pairs, 0, dev->stream_ws.total_bytes, dev->stream);
    cudaStreamSynchronize(dev->stream);
    if (st == 128) fail("index_out_of_range", "an index of a gather or an expert id of a matmul_id is out of range; the rows it selects were not computed");
    fail("backend", "a device-side wait gave up (status " + std::to_string(st) + "); the results of this call are invalid");
}

// (the caller holds dev->mu and has made the device current)
void execute_locked(lapid_b200_device *dev, const lapid_b200_launch *launches, size_t n, lapid_b200_buffer *const *buffers,
                    size_t nbuf, bool wait) {
    // Plan the activation pre-passes of the decode launches of this list:
    //  * launches that read the same A operand (q/k/v, gate/up) share one quantized copy, as long
    //    as no launch in between writes the buffer it comes from;
    //  * operands that no earlier launch of the list writes do not depend on anything in the
    //    list, so their pre-passes are hoisted into one batched launch at the head of the call
    //    and the GEMVs then follow each other directly.
    std::vector<ActSlot> slots;
    std::vector<int> slot_of(n, -1);
    size_t scratch_total = 0;
    {
        struct Range { const char *lo, *hi; };
        std::vector<Range> written;
        int last = -1;  // most recent slot, reusable by a non-hoisted launch
        for (size_t i = 0; i < n; i++) {
            const lapid_b200_launch &l = launches[i];
            if (l.kind == LAPID_B200_KERNEL_GATHER) {  // no scratch of its own; its output counts as written
                lapid_b200_buffer *gb = l.output < nbuf ? buffers[l.output] : nullptr;
                if (gb) {
                    written.push_back({(const char *)gb->ptr, (const char *)gb->ptr + gb->bytes});
                    if (last >= 0 && !slots[last].hoisted && (const char *)slots[last].ptr >= (const char *)gb->ptr &&
                        (const char *)slots[last].ptr < (const char *)gb->ptr + gb->bytes)
                        last = -1;
                }
                continue;
            }
            if (l.kind == LAPID_B200_KERNEL_MATMUL_ID && is_quant(l.b_dtype)) {  // a scratch slot of its own; its output counts as written
                ActSlot sl;
                sl.offset = scratch_total;
                scratch_total += plan_matmul_id(*dev, l).scratch;
                slots.push_back(sl);
                slot_of[i] = (int)slots.size() - 1;
                lapid_b200_buffer *gb = l.output < nbuf ? buffers[l.output] : nullptr;
                if (gb) {
                    written.push_back({(const char *)gb->ptr, (const char *)gb->ptr + gb->bytes});
                    if (last >= 0 && !slots[last].hoisted && (const char *)slots[last].ptr >= (const char *)gb->ptr &&
                        (const char *)slots[last].ptr < (const char *)gb->ptr + gb->bytes)
                        last = -1;
                }
                continue;
            }
            if (l.kind != LAPID_B200_KERNEL_MATMUL || !is_quant(l.b_dtype)) break;  // run_launch reports it
            Plan p = plan_launch(*dev, l);
            lapid_b200_buffer *ab = l.n_inputs > 0 && l.inputs[0] < nbuf ? buffers[l.inputs[0]] : nullptr;
            lapid_b200_buffer *ob = l.output < nbuf ? buffers[l.output] : nullptr;
            if (p.gemv && ab && l.a_dtype != LAPID_B200_DTYPE_ACT_Q8) {
                ActSlot key;
                key.ptr = ab->ptr;
                key.off = l.a.offset;
                key.bs = l.a.batch_stride;
                key.rs = l.a.row_stride;
                key.rows = p.rows;
                key.m = (uint32_t)l.m;
                key.k = (uint32_t)l.k;
                key.records = p.records();
                key.a_type = act_type_of(l.a_dtype);
                bool clean = true;  // nothing in the list so far wrote the buffer A lives in
                for (const Range &w : written)
                    if ((const char *)ab->ptr < w.hi && w.lo < (const char *)ab->ptr + ab->bytes) clean = false;
                // Option (off): two rows of Q4_K whose activations come from the pre-pass at the head on the dp4a kernel.
                // It used to beat the tensor-core kernel there; since the balanced-stream kernel the tensor-core
                // kernels win (the sweep step of 16 launches: 76.7 against 86.3 us)
                if (clean && dev->two_row_dp4a && dev->act_reuse && dev->early_acts && dev->pdl && p.rows == 2 && p.mma && p.fast &&
                    l.b_dtype == LAPID_B200_DTYPE_Q4_K)
                    key.records = 1;
                int found = -1;
                if (dev->act_reuse) {
                    if (clean) {
                        for (size_t s2 = 0; s2 < slots.size(); s2++)
                            if (slots[s2].hoisted && slots[s2].same(key)) found = (int)s2;
                    } else if (last >= 0 && slots[last].same(key) && !slots[last].hoisted) {
                        found = last;  // same operand as the launch right before, not rewritten since (checked below)
                    }
                }
                if (found < 0) {
                    key.hoisted = clean && dev->act_reuse;
                    key.offset = scratch_total;
                    scratch_total += p.scratch;
                    slots.push_back(key);
                    found = (int)slots.size() - 1;
                }
                slot_of[i] = found;
                last = found;
            }
            if (p.tc) {
                ActSlot sl;
                sl.offset = scratch_total;
                scratch_total += p.scratch;
                slots.push_back(sl);
                slot_of[i] = (int)slots.size() - 1;
            }
            if (ob && !p.noop) {
                written.push_back({(const char *)ob->ptr, (const char *)ob->ptr + ob->bytes});
                // a write into the buffer the latest non-hoisted slot was read from invalidates it
                if (last >= 0 && !slots[last].hoisted && (const char *)slots[last].ptr >= (const char *)ob->ptr &&
                    (const char *)slots[last].ptr < (const char *)ob->ptr + ob->bytes)
                    last = -1;
            }
        }
    }
    dev->ensure_scratch(scratch_total);
    struct HoistScope {  // after_hoist is meaningful inside this list only
        lapid_b200_device *d;
        explicit HoistScope(lapid_b200_device *dev_) : d(dev_) { d->after_hoist = -1; }
        ~HoistScope() { d->after_hoist = -1; }
    } hoist_scope(dev);
    // Operands quantized by their producer (ACT_Q8) were complete before this list began, like the results of
    // the pre-pass at its head: with the first kernel of the list fully serialised, the later ones may read them early.
    if (dev->early_acts && dev->pdl)
        for (size_t i = 0; i < n; i++)
            if (launches[i].kind == LAPID_B200_KERNEL_MATMUL && launches[i].a_dtype == LAPID_B200_DTYPE_ACT_Q8) dev->after_hoist = 0;
    {
        lb::ActQuantBatch batch;
        batch.count = 0;
        uint64_t groups = 0;
        auto flush = [&]() {
            if (batch.count == 0) return;
            cuda_check(lb::launch_act_quant_batch(batch, dev->sm_count, dev->pdl, dev->stream), "act_quant launch");
            dev->launches++;
            if (dev->early_acts) dev->after_hoist = 0;
            batch.count = 0;
            groups = 0;
        };
        for (ActSlot &sl : slots) {
            if (!sl.hoisted) continue;
            char *base = (char *)dev->scratch + sl.offset;
            size_t qa_b = align_up((uint64_t)sl.rows * sl.k, 256), sc_b = align_up((uint64_t)sl.rows * (sl.k / 32) * 4, 256);
            lb::ActQuantArgs &q = batch.item[batch.count];
            q = lb::ActQuantArgs{};
            q.a = sl.ptr;
            q.a_type = sl.a_type;
            q.a_off = sl.off;
            q.a_bs = sl.bs;
            q.a_rs = sl.rs;
            q.rows = sl.rows;
            q.m = sl.m;
            q.k = sl.k;
            q.qa = (int8_t *)base;
            q.da = (float *)(base + qa_b);
            q.bs = (float *)(base + qa_b + sc_b);  // written for every format; only Q4_K reads it
            q.records = sl.records;
            groups += (uint64_t)sl.rows * (sl.k / 32);
            batch.group_end[batch.count] = groups;
            batch.count++;
            sl.done = true;
            if (batch.count == lb::ACT_BATCH_MAX) flush();
        }
        flush();
    }
    PendingGroup pend;
    pend.split_early = n >= 8;
    PendingGroup *pp = dev->gemv_group && !dev->profile ? &pend : nullptr;
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(dev->stream, &capturing);
    const bool profiling = dev->profile && capturing == cudaStreamCaptureStatusNone;  // (events of a capture cannot be timed)
    if (profiling)
        while (dev->profile_events.size() < 2 * n) {
            cudaEvent_t e;
            cuda_check(cudaEventCreate(&e), "cudaEventCreate");
            dev->profile_events.push_back(e);
        }
    try {
        for (size_t i = 0; i < n; i++) {
            if (profiling) cuda_check(cudaEventRecord(dev->profile_events[2 * i], dev->stream), "cudaEventRecord");
            run_launch(*dev, launches[i], buffers, nbuf, slot_of[i] >= 0 ? &slots[slot_of[i]] : nullptr, pp);
            if (profiling) cuda_check(cudaEventRecord(dev->profile_events[2 * i + 1], dev->stream), "cudaEventRecord");
        }
    } catch (...) {
        pend.flush(*dev);  // the launches before the rejected one still run, as they would one by one
        throw;
    }
    pend.flush(*dev);
    if (wait || profiling) {
        cuda_check(cudaStreamSynchronize(dev->stream), "cudaStreamSynchronize");
        if (profiling)
            for (size_t i = 0; i < n; i++) {
                float ms = 0.0f;
                if (cudaEventElapsedTime(&ms, dev->profile_events[2 * i], dev->profile_events[2 * i + 1]) != cudaSuccess) continue;
                const lapid_b200_launch &l = launches[i];
                const char *kind = l.kind == LAPID_B200_KERNEL_GATHER ? "gather" : l.kind == LAPID_B200_KERNEL_MATMUL_ID ? "matmul_id"
                                   : l.batch * l.m <= dev->gemv_max_rows ? "matmul_decode" : "matmul_prefill";
                auto &e = dev->profile_by_kind[kind];
                e.first++;
                e.second += ms;
            }
        check_status_word(dev);
    }
}

void execute_impl(lapid_b200_device *dev, const lapid_b200_launch *launches, size_t n, lapid_b200_buffer *const *buffers,
                  size_t nbuf, bool wait) {
    need(dev);
    if (n && !launches) fail("invalid_argument", "launches is NULL");
    if (nbuf && !buffers) fail("invalid_argument", "buffers is NULL");
    std::lock_guard<std::mutex> lock(dev->mu);
    dev->make_current();
    execute_locked(dev, launches, n, buffers, nbuf, wait);
}

// Byte range of buffer `b` that launch `l` reads as its A operand / gather ids / x (`in`) or writes (`!in`);
// false when the launch does not touch the buffer that way. Conservative: whole buffers for the launch kinds whose
// views are not simple matrices.
bool launch_range(const lapid_b200_launch &l, uint32_t b, bool in, uint64_t buf_bytes, uint64_t &lo, uint64_t &hi) {
    auto span = [&](const lapid_b200_matview &v, uint64_t width, uint64_t elem) {
        const uint64_t batch = l.batch ? l.batch : 1, m = l.m ? l.m : 1;
        lo = v.offset * elem;
        hi = (v.offset + (batch - 1) * v.batch_stride + (m - 1) * v.row_stride + width) * elem;
    };
    if (in) {
        bool hit = false;
        for (int i = 0; i < l.n_inputs && i < 3; i++) hit = hit || l.inputs[i] == b;
        if (!hit) return false;
        lo = 0, hi = buf_bytes;
        if (l.kind == LAPID_B200_KERNEL_MATMUL && l.n_inputs >= 1 && l.inputs[0] == b && (l.n_inputs < 2 || l.inputs[1] != b) &&
            (l.n_inputs < 3 || l.inputs[2] != b) && is_act_float(l.a_dtype))
            span(l.a, l.k, act_elem_size(l.a_dtype));
        return true;
    }
    if (l.output != b) return false;
    lo = 0, hi = buf_bytes;
    if (l.kind == LAPID_B200_KERNEL_MATMUL) span(l.out, l.n, 4);
    return true;
}

// write + execute + read of one step as one pipelined call (see the header).
void execute_io_impl(lapid_b200_device *dev, const lapid_b200_launch *launches, size_t n, lapid_b200_buffer *const *buffers, size_t nbuf,
                     const lapid_b200_io *writes, size_t n_writes, const lapid_b200_io *reads, size_t n_reads, size_t chunk) {
    need(dev);
    if (n && !launches) fail("invalid_argument", "launches is NULL");
    if (nbuf && !buffers) fail("invalid_argument", "buffers is NULL");
    if ((n_writes && !writes) || (n_reads && !reads)) fail("invalid_argument", "writes or reads is NULL");
    // Chunk boundaries: `chunk` launches each, or (0) up to three chunks holding about the same number of transferred
    // bytes each, by the launches the transfers are tied to -- the first upload and the last download are the copies
    // nothing hides, so neither the first nor the last chunk should carry most of the bytes.
    std::vector<size_t> first_of;  // first launch of every chunk, then n
    if (chunk) {
        for (size_t f = 0; f < n; f += chunk) first_of.push_back(f);
    } else if (n) {
        std::vector<uint64_t> bytes_at(n, 0);
        uint64_t total = 0;
        for (size_t i = 0; i < n_writes; i++)
            if (writes[i].launch < n) bytes_at[writes[i].launch] += writes[i].bytes, total += writes[i].bytes;
        for (size_t i = 0; i < n_reads; i++)
            if (reads[i].launch < n) bytes_at[reads[i].launch] += reads[i].bytes, total += reads[i].bytes;
        const size_t want = n >= 6 && total >= (1u << 20) ? 3 : (n >= 2 && total >= (256u << 10) ? 2 : 1);
        first_of.push_back(0);
        uint64_t run = 0;
        for (size_t i = 0; i + 1 < n && first_of.size() < want; i++) {
            run += bytes_at[i];
            if (run * want >= total * first_of.size()) first_of.push_back(i + 1);
        }
    }
    const size_t n_chunks = first_of.size();
    first_of.push_back(n);
    std::vector<uint32_t> chunk_of(n, 0);
    for (size_t c = 0; c < n_chunks; c++)
        for (size_t i = first_of[c]; i < first_of[c + 1]; i++) chunk_of[i] = (uint32_t)c;
    auto check_io = [&](const lapid_b200_io &io, const char *what) {
        if (io.buffer >= nbuf || !buffers[io.buffer])
            fail("invalid_launch", std::string("execute_io: ") + what + " names buffer " + std::to_string(io.buffer) + " of " + std::to_string(nbuf));
        if (buffers[io.buffer]->dev != dev) fail("wrong_backend", std::string("execute_io: ") + what + " buffer belongs to another device");
        if (io.bytes && !io.host) fail("invalid_argument", std::string("execute_io: ") + what + " host pointer is NULL");
        if (io.offset > buffers[io.buffer]->bytes || io.bytes > buffers[io.buffer]->bytes - io.offset)
            fail("out_of_bounds", std::string("execute_io: ") + what + " of " + std::to_string(io.bytes) + " bytes at " + std::to_string(io.offset) +
                                      " in a buffer of " + std::to_string(buffers[io.buffer]->bytes));
        if (n && io.launch >= n) fail("invalid_launch", std::string("execute_io: ") + what + " names launch " + std::to_string(io.launch) + " of " + std::to_string(n));
    };
    // A write is uploaded just before the chunk of the launch it names: no launch of an earlier chunk may read or
    // write what it brings. A read is downloaded right after the chunk of the launch it names: no launch of a
    // later chunk may write what it takes.
    for (size_t i = 0; i < n_writes; i++) {
        check_io(writes[i], "write");
        for (size_t j = 0; n && j < first_of[chunk_of[writes[i].launch]]; j++) {
            uint64_t lo, hi;
            for (int in = 0; in < 2; in++)
                if (launch_range(launches[j], writes[i].buffer, in != 0, buffers[writes[i].buffer]->bytes, lo, hi) && lo < writes[i].offset + writes[i].bytes &&
                    writes[i].offset < hi)
                    fail("invalid_launch", "execute_io: write " + std::to_string(i) + " is tied to launch " + std::to_string(writes[i].launch) +
                                               " but launch " + std::to_string(j) + " of an earlier chunk uses that memory");
        }
    }
    for (size_t i = 0; i < n_reads; i++) {
        check_io(reads[i], "read");
        for (size_t j = n ? first_of[chunk_of[reads[i].launch] + 1] : 0; j < n; j++) {
            uint64_t lo, hi;
            if (launch_range(launches[j], reads[i].buffer, false, buffers[reads[i].buffer]->bytes, lo, hi) && lo < reads[i].offset + reads[i].bytes &&
                reads[i].offset < hi)
                fail("invalid_launch", "execute_io: read " + std::to_string(i) + " is tied to launch " + std::to_string(reads[i].launch) +
                                           " but launch " + std::to_string(j) + " of a later chunk writes that memory");
        }
    }
    std::lock_guard<std::mutex> lock(dev->mu);
    dev->make_current();
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(dev->stream, &capturing);
    if (capturing != cudaStreamCaptureStatusNone) fail("invalid_launch", "execute_io waits for its copies: not inside a stream capture");
    if (!dev->io_in) cuda_check(cudaStreamCreateWithFlags(&dev->io_in, cudaStreamNonBlocking), "cudaStreamCreate");
    if (!dev->io_out) cuda_check(cudaStreamCreateWithFlags(&dev->io_out, cudaStreamNonBlocking), "cudaStreamCreate");
    while (dev->io_events.size() < 2 * n_chunks + 1) {
        cudaEvent_t e;
        cuda_check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
        dev->io_events.push_back(e);
    }
    // the copies start behind whatever is already queued on the device's stream
    cudaEvent_t start = dev->io_events[2 * n_chunks];
    cuda_check(cudaEventRecord(start, dev->stream), "cudaEventRecord");
    cuda_check(cudaStreamWaitEvent(dev->io_in, start, 0), "cudaStreamWaitEvent");
    cuda_check(cudaStreamWaitEvent(dev->io_out, start, 0), "cudaStreamWaitEvent");
    auto finish = [&]() {  // leave nothing in flight, whatever happened
        cudaStreamSynchronize(dev->io_in);
        cudaStreamSynchronize(dev->stream);
        cudaStreamSynchronize(dev->io_out);
    };
    try {
        // Transfers of one chunk that continue each other in the buffer and in host memory go as one copy (a copy
        // costs microseconds of host time to queue, whatever its size).
        auto copies_of = [&](const lapid_b200_io *ios, size_t count, size_t c) {
            std::vector<lapid_b200_io> v;
            for (size_t i = 0; i < count; i++)
                if ((n ? chunk_of[ios[i].launch] : 0) == c && ios[i].bytes) v.push_back(ios[i]);
            std::sort(v.begin(), v.end(), [](const lapid_b200_io &a, const lapid_b200_io &b) {
                return a.buffer != b.buffer ? a.buffer < b.buffer : a.offset < b.offset;
            });
            std::vector<lapid_b200_io> out;
            for (const lapid_b200_io &io : v) {
                if (!out.empty() && out.back().buffer == io.buffer && out.back().offset + out.back().bytes == io.offset &&
                    (char *)out.back().host + out.back().bytes == (char *)io.host)
                    out.back().bytes += io.bytes;
                else
                    out.push_back(io);
            }
            return out;
        };
        // all uploads are queued now, in chunk order: chunk c + 1 arrives while chunk c computes
        for (size_t c = 0; c < (n_chunks ? n_chunks : 1); c++) {
            for (const lapid_b200_io &w : copies_of(writes, n_writes, c))
                cuda_check(cudaMemcpyAsync((char *)buffers[w.buffer]->ptr + w.offset, w.host, w.bytes, cudaMemcpyHostToDevice, dev->io_in),
                           "execute_io upload");
            if (n_chunks) cuda_check(cudaEventRecord(dev->io_events[2 * c], dev->io_in), "cudaEventRecord");
        }
        for (size_t c = 0; c < n_chunks; c++) {
            const size_t first = first_of[c], count = first_of[c + 1] - first;
            cuda_check(cudaStreamWaitEvent(dev->stream, dev->io_events[2 * c], 0), "cudaStreamWaitEvent");
            execute_locked(dev, launches + first, count, buffers, nbuf, false);
            cuda_check(cudaEventRecord(dev->io_events[2 * c + 1], dev->stream), "cudaEventRecord");
            cuda_check(cudaStreamWaitEvent(dev->io_out, dev->io_events[2 * c + 1], 0), "cudaStreamWaitEvent");
            for (const lapid_b200_io &r : copies_of(reads, n_reads, c))
                cuda_check(cudaMemcpyAsync(r.host, (const char *)buffers[r.buffer]->ptr + r.offset, r.bytes, cudaMemcpyDeviceToHost, dev->io_out),
                           "execute_io download");
        }
        if (!n_chunks) {  // no launches: the writes, then the reads
            cuda_check(cudaStreamSynchronize(dev->io_in), "execute_io");
            for (size_t i = 0; i < n_reads; i++)
                if (reads[i].bytes)
                    cuda_check(cudaMemcpyAsync(reads[i].host, (const char *)buffers[reads[i].buffer]->ptr + reads[i].offset, reads[i].bytes,
                                               cudaMemcpyDeviceToHost, dev->io_out), "execute_io download");
        }
    } catch (...) {
        finish();
        throw;
    }
    cuda_check(cudaStreamSynchronize(dev->io_in), "execute_io");
    cuda_check(cudaStreamSynchronize(dev->stream), "execute_io");
    cuda_check(cudaStreamSynchronize(dev->io_out), "execute_io");
    check_status_word(dev);
}

}  // namespace

struct lapid_b200_tp_comm {
    lapid_b200_device *dev = nullptr;  // retained
    lb::TpAllReduceArgs args{};
};

namespace lb {
// For entry points defined in other files: records the error for lapid_b200_last_error() and
// returns its status code.
int32_t report_error(const char *code, const std::string &message) { return record(Error{code, message}); }
}  // namespace lb

// ================================================================== extern "C"
extern "C" {

uint32_t lapid_b200_abi_version(void) { return LAPID_B200_ABI_VERSION; }

lapid_b200_status lapid_b200_check_abi(uint32_t expected) {
    return guard([&] {
        if (expected != LAPID_B200_ABI_VERSION)
            fail("abi_mismatch", "header ABI " + std::to_string(expected) + ", library ABI " + std::to_string(LAPID_B200_ABI_VERSION));
    });
}

const char *lapid_b200_last_error(void) { return g_has_error ? g_last_error.c_str() : nullptr; }

lapid_b200_status lapid_b200_device_open(int32_t ordinal, lapid_b200_device **out) {
    return guard([&] {
        if (!out) fail("invalid_argument", "out is NULL");
        int count = 0;
        cudaError_t e = cudaGetDeviceCount(&count);
        if (e != cudaSuccess || count == 0)
            fail("cuda_unavailable", std::string("no CUDA device: ") + (e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e)));
        if (ordinal < 0 || ordinal >= count)
            fail("device_unavailable", "CUDA device " + std::to_string(ordinal) + " does not exist (" + std::to_string(count) + " devices)");
        cudaDeviceProp prop{};
        cuda_check(cudaGetDeviceProperties(&prop, ordinal), "cudaGetDeviceProperties");
        if (prop.major != 10)
            fail("device_unavailable", std::string(prop.name) + " is compute capability " + std::to_string(prop.major) + "." +
                                           std::to_string(prop.minor) + "; this library carries sm_100a code only");
        auto *d = new lapid_b200_device();
        d->ordinal = ordinal;
        d->sm_count = prop.multiProcessorCount;
        d->name = prop.name;
        try {
            d->make_current();
            cuda_check(cudaStreamCreateWithFlags(&d->own_stream, cudaStreamNonBlocking), "cudaStreamCreate");
            d->stream = d->own_stream;
            cuda_check(cudaHostAlloc((void **)&d->status_host, sizeof(int), cudaHostAllocMapped), "cudaHostAlloc");
            *d->status_host = 0;
            cuda_check(cudaHostGetDevicePointer((void **)&d->status_dev, d->status_host, 0), "cudaHostGetDevicePointer");
            const size_t ws_bytes = lb::qgemv_kq_stream_ws_bytes(d->sm_count, &d->stream_ws);
            void *ws = nullptr;
            cuda_check(cudaMalloc(&ws, ws_bytes), "cudaMalloc(decode workspace)");
            d->stream_ws.pairs = (uint2 *)ws;
            d->stream_ws.stage = (uint8_t *)ws + d->stream_ws.n_pairs * 8;
            cuda_check(cudaMemset(ws, 0, ws_bytes), "cudaMemset(decode workspace)");
            cuda_check(lb::iq_grids_upload(), "i-quant codebook upload");
        } catch (...) {
            delete d;
            throw;
        }
        *out = d;
    });
}

void lapid_b200_device_retain(lapid_b200_device *dev) {
    if (dev) dev->refs.fetch_add(1);
}
void lapid_b200_device_free(lapid_b200_device *dev) { device_release(dev); }

lapid_b200_status lapid_b200_device_name(const lapid_b200_device *dev, char *out, size_t cap) {
    return guard([&] {
        if (!dev || !out || cap == 0) fail("invalid_argument", "device, out or cap is NULL/0");
        std::string s = dev->name + " (sm_100a, " + std::to_string(dev->sm_count) + " SMs)";
        size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
        std::memcpy(out, s.data(), n);
        out[n] = 0;
    });
}

lapid_b200_status lapid_b200_device_set_stream(lapid_b200_device *dev, void *cuda_stream) {
    return guard([&] {
        need(dev);
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->stream = cuda_stream ? (cudaStream_t)cuda_stream : dev->own_stream;
    });
}

lapid_b200_status lapid_b200_device_synchronize(lapid_b200_device *dev) {
    return guard([&] {
        need(dev);
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        cuda_check(cudaStreamSynchronize(dev->stream), "cudaStreamSynchronize");
        check_status_word(dev);
    });
}

lapid_b200_status lapid_b200_device_set_option(lapid_b200_device *dev, const char *key, const char *value) {
    return guard([&] {
        need(dev);
        if (!key || !value) fail("invalid_argument", "key or value is NULL");
        std::lock_guard<std::mutex> lock(dev->mu);
        std::string k = key, v = value;
        if (k == "pdl") {
            dev->pdl = v != "0";
        } else if (k == "early_acts") {
            dev->early_acts = v != "0";
        } else if (k == "tp_spin_limit") {
            long r = std::atol(value);
            if (r < 0 || r > (1l << 30)) fail("invalid_argument", "tp_spin_limit must be in 0..2^30 (0 = the default)");
            dev->tp_spin_limit = (uint32_t)r;
        } else if (k == "gemv_max_rows") {
            int r = std::atoi(value);
            if (r < 0 || r > 8) fail("invalid_argument", "gemv_max_rows must be in 0..8");
            dev->gemv_max_rows = (uint32_t)r;
        } else if (k == "gemv") {
            if (v == "fast") dev->gemv_fast = true;
            else if (v == "generic") dev->gemv_fast = false;
            else fail("invalid_argument", "gemv must be \"fast\" or \"generic\"");
        } else if (k == "act_reuse") {
            dev->act_reuse = v != "0";
        } else if (k == "gemv_group") {
            dev->gemv_group = v != "0";
        } else if (k == "gemv_mma_rows") {
            int r = std::atoi(value);
            if (r < 0 || r > 8) fail("invalid_argument", "gemv_mma_rows must be in 0..8");
            dev->gemv_mma_rows = (uint32_t)r;
        } else if (k == "gemv_stream") {
            int r = std::atoi(value);
            if (r < 0 || r > 2) fail("invalid_argument", "gemv_stream must be 0 (never), 1 (Q5_K) or 2 (Q4_K and Q5_K)");
            dev->gemv_stream = r;
        } else if (k == "gemv_small_dp4a") {
            dev->small_dp4a = std::atoi(value) != 0;
        } else if (k == "gemv_stream_config") {
            lb::qgemv_kq_stream_set_config(std::atoi(value));
        } else if (k == "gemv_stream_ctas") {
            lb::qgemv_kq_stream_set_ctas_per_sm(std::atoi(value));
        } else if (k == "gemv_stream_early_ctas") {
            lb::qgemv_kq_stream_set_early_ctas(std::atoi(value));
        } else if (k == "profile") {
            dev->profile = v != "0";
            if (!dev->profile) dev->profile_by_kind.clear();
        } else if (k == "gemv_stream_spin_limit") {
            lb::qgemv_kq_stream_set_spin_limit(std::atoi(value));
        } else if (k == "gemv_stream_big_units") {
            lb::qgemv_kq_stream_set_big_units(std::atoi(value));
        } else if (k == "gemv_stream_final_tiles") {
            lb::qgemv_kq_stream_set_final_tiles(std::atoi(value));
        } else if (k == "gemv_stream_debug") {
            lb::qgemv_kq_stream_set_debug(std::atoi(value));
        } else if (k == "gemv_two_row_dp4a") {
            dev->two_row_dp4a = v != "0";
        } else if (k == "gemv_mma_config") {
            lb::qgemv_q4k_mma_set_config(std::atoi(value));
        } else if (k == "gemv_q6k_mma_config") {
            lb::qgemv_q6k_mma_set_config(std::atoi(value));
        } else if (k == "gemv_mxfp4_mma_rows") {
            int r = std::atoi(value);
            if (r < 0 || r > 8) fail("invalid_argument", "gemv_mxfp4_mma_rows must be in 0..8");
            dev->mxfp4_mma_rows = (uint32_t)r;
        } else if (k == "gemv_mxfp4_k_split") {
            lb::qgemv_mxfp4_set_k_split(std::atoi(value));
        } else if (k == "gemv_mxfp4_staged") {
            lb::qgemv_mxfp4_set_staged(std::atoi(value));
        } else if (k == "gemv_iq_k_split") {
            lb::qgemv_iq_set_k_split(std::atoi(value));
        } else if (k == "gemv_iq_rows") {  // weight rows per warp of the i-quant decode kernel: 1, 2 (0: per launch)
            lb::qgemv_iq_set_rows_per_warp(std::atoi(value));
        } else if (k == "gemv_ctas_per_sm") {
            lb::qgemv_q4k_fast_set_cta_cap(std::atoi(value));
        } else if (k == "gemm_wide") {
            lb::qgemm_tc_set_wide(std::atoi(value));
        } else if (k == "gemm_splitk") {
            lb::qgemm_tc_set_splitk(std::atoi(value));
        } else if (k == "gemm_pair") {
            lb::qgemm_tc_set_pair(std::atoi(value));
        } else if (k == "gemm_tall") {
            lb::qgemm_tc_set_tall(std::atoi(value));
        } else if (k == "gemm") {
            if (v == "f32") dev->gemm_f32 = true;
            else if (v == "tc") dev->gemm_f32 = false;
            else fail("invalid_argument", "gemm must be \"tc\" or \"f32\"");
        } else {
            fail("invalid_argument", "unknown option \"" + k + "\"");
        }
    });
}

lapid_b200_status lapid_b200_alloc(lapid_b200_device *dev, size_t bytes, lapid_b200_buffer **out) {
    return guard([&] {
        need(dev);
        if (!out) fail("invalid_argument", "out is NULL");
        dev->make_current();
        void *p = nullptr;
        cuda_check(cudaMalloc(&p, bytes ? bytes : 1), "cudaMalloc");
        *out = new_buffer(dev, p, bytes, true);
    });
}

lapid_b200_status lapid_b200_upload(lapid_b200_device *dev, const void *host, size_t bytes, lapid_b200_buffer **out) {
    return guard([&] {
        need(dev);
        if (!out || (bytes && !host)) fail("invalid_argument", "out or host is NULL");
        dev->make_current();
        void *p = nullptr;
        cuda_check(cudaMalloc(&p, bytes ? bytes : 1), "cudaMalloc");
        cudaError_t e = cudaSuccess;
        {
            std::lock_guard<std::mutex> lock(dev->mu);
            if (bytes) e = cudaMemcpyAsync(p, host, bytes, cudaMemcpyHostToDevice, dev->stream);
            if (e == cudaSuccess) e = cudaStreamSynchronize(dev->stream);  // `host` may be reused on return
        }
        if (e != cudaSuccess) {
            cudaFree(p);
            cuda_check(e, "upload");
        }
        *out = new_buffer(dev, p, bytes, true);
    });
}

lapid_b200_status lapid_b200_wrap(lapid_b200_device *dev, void *device_ptr, size_t bytes, lapid_b200_buffer **out) {
    return guard([&] {
        need(dev);
        if (!out || !device_ptr) fail("invalid_argument", "out or device_ptr is NULL");
        if ((uintptr_t)device_ptr & 15) fail("invalid_argument", "wrapped device memory must be 16-byte aligned");
        *out = new_buffer(dev, device_ptr, bytes, false);
    });
}

lapid_b200_status lapid_b200_write(lapid_b200_buffer *buf, size_t offset, const void *host, size_t bytes) {
    return guard([&] {
        need(buf, "buffer");
        if (bytes && !host) fail("invalid_argument", "host is NULL");
        if (offset > buf->bytes || bytes > buf->bytes - offset)
            fail("out_of_bounds", "write of " + std::to_string(bytes) + " bytes at " + std::to_string(offset) + " into a buffer of " +
                                      std::to_string(buf->bytes));
        if (!bytes) return;
        lapid_b200_device *dev = buf->dev;
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        cuda_check(cudaMemcpyAsync((char *)buf->ptr + offset, host, bytes, cudaMemcpyHostToDevice, dev->stream), "write");
        // pageable memory is staged before the call returns; pinned memory must stay valid until
        // the copy ran, so wait: `host` may be reused when this returns (Backend::write contract)
        cuda_check(cudaStreamSynchronize(dev->stream), "write");
    });
}

lapid_b200_status lapid_b200_download(lapid_b200_buffer *buf, void *host, size_t bytes) {
    return guard([&] {
        need(buf, "buffer");
        if (bytes && !host) fail("invalid_argument", "host is NULL");
        if (bytes > buf->bytes)
            fail("out_of_bounds", "download of " + std::to_string(bytes) + " bytes from a buffer of " + std::to_string(buf->bytes));
        lapid_b200_device *dev = buf->dev;
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        if (bytes) cuda_check(cudaMemcpyAsync(host, buf->ptr, bytes, cudaMemcpyDeviceToHost, dev->stream), "download");
        cuda_check(cudaStreamSynchronize(dev->stream), "download");
    });
}

void lapid_b200_buffer_retain(lapid_b200_buffer *buf) {
    if (buf) buf->refs.fetch_add(1);
}
void lapid_b200_buffer_free(lapid_b200_buffer *buf) { buffer_release(buf); }
size_t lapid_b200_buffer_size(const lapid_b200_buffer *buf) { return buf ? buf->bytes : 0; }
void *lapid_b200_buffer_device_ptr(const lapid_b200_buffer *buf) { return buf ? buf->ptr : nullptr; }

lapid_b200_status lapid_b200_prepare(lapid_b200_device *dev, const lapid_b200_launch *launches, size_t n) {
    return guard([&] {
        need(dev);
        if (n && !launches) fail("invalid_argument", "launches is NULL");
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        size_t scratch = 0;  // every decode launch may get its own slot (see execute)
        for (size_t i = 0; i < n; i++) {
            if (launches[i].kind == LAPID_B200_KERNEL_GATHER) check_gather(launches[i]);
            else if (launches[i].kind == LAPID_B200_KERNEL_MATMUL_ID) scratch += plan_matmul_id(*dev, launches[i]).scratch;
            else scratch += plan_launch(*dev, launches[i]).scratch;
        }
        dev->ensure_scratch(scratch);
    });
}

lapid_b200_status lapid_b200_execute(lapid_b200_device *dev, const lapid_b200_launch *launches, size_t n,
                                     lapid_b200_buffer *const *buffers, size_t nbuf) {
    return guard([&] { execute_impl(dev, launches, n, buffers, nbuf, true); });
}

lapid_b200_status lapid_b200_execute_async(lapid_b200_device *dev, const lapid_b200_launch *launches, size_t n,
                                           lapid_b200_buffer *const *buffers, size_t nbuf) {
    return guard([&] { execute_impl(dev, launches, n, buffers, nbuf, false); });
}

lapid_b200_status lapid_b200_execute_io(lapid_b200_device *dev, const lapid_b200_launch *launches, size_t n, lapid_b200_buffer *const *buffers,
                                        size_t nbuf, const lapid_b200_io *writes, size_t n_writes, const lapid_b200_io *reads, size_t n_reads,
                                        size_t chunk) {
    return guard([&] { execute_io_impl(dev, launches, n, buffers, nbuf, writes, n_writes, reads, n_reads, chunk); });
}

uint64_t lapid_b200_take_launch_count(lapid_b200_device *dev) { return dev ? dev->launches.exchange(0) : 0; }

lapid_b200_status lapid_b200_take_profile(lapid_b200_device *dev, lapid_b200_profile_entry *entries, size_t cap, size_t *n) {
    return guard([&] {
        need(dev);
        if (!n || (cap && !entries)) fail("invalid_argument", "n or entries is NULL");
        std::lock_guard<std::mutex> lock(dev->mu);
        std::vector<std::pair<std::string, std::pair<uint64_t, double>>> v(dev->profile_by_kind.begin(), dev->profile_by_kind.end());
        std::sort(v.begin(), v.end(), [](const auto &a, const auto &b) { return a.second.second > b.second.second; });
        *n = v.size();
        if (cap < v.size()) return;  // (the caller asks again with room; nothing is drained)
        for (size_t i = 0; i < v.size(); i++) {
            std::snprintf(entries[i].kind, sizeof(entries[i].kind), "%s", v[i].first.c_str());
            entries[i].launches = v[i].second.first;
            entries[i].ms = v[i].second.second;
        }
        dev->profile_by_kind.clear();
    });
}

lapid_b200_status lapid_b200_decode_trace_begin(lapid_b200_device *dev, uint32_t launches) {
    return guard([&] {
        need(dev);
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        cuda_check(cudaStreamSynchronize(dev->stream), "cudaStreamSynchronize");
        cuda_check(lb::qgemv_kq_stream_trace_begin(launches, dev->sm_count), "trace buffer");
    });
}

lapid_b200_status lapid_b200_decode_trace_read(lapid_b200_device *dev, uint64_t *out, uint64_t cap_words, uint32_t *launches, uint32_t *ctas) {
    return guard([&] {
        need(dev);
        if (!launches || !ctas) fail("invalid_argument", "launches or ctas is NULL");
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        cuda_check(cudaStreamSynchronize(dev->stream), "cudaStreamSynchronize");
        *launches = lb::qgemv_kq_stream_trace_read((unsigned long long *)out, cap_words, ctas);
    });
}

lapid_b200_status lapid_b200_quant_layout(int32_t format, uint64_t rows, uint64_t cols, lapid_b200_layout *out) {
    return guard([&] {
        if (!out) fail("invalid_argument", "out is NULL");
        *out = layout_of(format, rows, cols);
    });
}

lapid_b200_status lapid_b200_dequantize(lapid_b200_device *dev, int32_t format, const lapid_b200_buffer *src, uint64_t rows,
                                        uint64_t cols, lapid_b200_buffer *dst) {
    return guard([&] {
        need(dev);
        if (!src || !dst) fail("invalid_argument", "src or dst is NULL");
        if (cols == 0) fail("invalid_launch", "quantized cols must be positive");
        lapid_b200_layout l = layout_of(format, rows, cols);
        if (src->bytes < l.scales_offset + l.scales_bytes)
            fail("out_of_bounds", "dequantize: buffer too small (" + std::to_string(src->bytes) + " < " + std::to_string(l.total) + ")");
        if (dst->bytes / 4 < rows * cols)
            fail("out_of_bounds", "dequantize: out has " + std::to_string(dst->bytes / 4) + " elements, expected " + std::to_string(rows * cols));
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        cuda_check(lb::launch_dequantize(format, src->ptr, rows, cols, l.scales_offset, (float *)dst->ptr, dev->sm_count, dev->stream),
                   "dequantize launch");
        dev->launches++;
        cuda_check(cudaStreamSynchronize(dev->stream), "dequantize");
    });
}

lapid_b200_status lapid_b200_quantize(lapid_b200_device *dev, int32_t format, const lapid_b200_buffer *src, uint64_t rows,
                                      uint64_t cols, lapid_b200_buffer *dst) {
    return guard([&] {
        need(dev);
        if (!src || !dst) fail("invalid_argument", "src or dst is NULL");
        if (cols == 0) fail("invalid_launch", "quantized cols must be positive");
        if (is_iquant(format))
            fail("unsupported", "quantize: the i-quant quantizers (lattice searches) are not built; import blocks with from_ggml_blocks");
        lapid_b200_layout l = layout_of(format, rows, cols);
        if (src->bytes / 4 < rows * cols)
            fail("shape_mismatch", "quantize: data has " + std::to_string(src->bytes / 4) + " elements, expected " +
                                       std::to_string(rows) + "x" + std::to_string(cols));
        if (dst->bytes < l.total)
            fail("out_of_bounds", "quantize: output holds " + std::to_string(dst->bytes) + " < " + std::to_string(l.total) + " bytes");
        if (((uintptr_t)src->ptr & 15) != 0) fail("invalid_launch", "quantize: source must be 16-byte aligned");
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        cuda_check(lb::launch_quantize(format, (const float *)src->ptr, rows, cols, l.scales_offset, l.total, dst->ptr, dev->sm_count,
                                       dev->stream),
                   "quantize launch");
        dev->launches++;
        cuda_check(cudaStreamSynchronize(dev->stream), "quantize");
    });
}

lapid_b200_status lapid_b200_from_ggml_blocks(lapid_b200_device *dev, int32_t format, const lapid_b200_buffer *src,
                                              uint64_t src_bytes, uint64_t rows, uint64_t cols, lapid_b200_buffer *dst) {
    return guard([&] {
        need(dev);
        if (!src || !dst) fail("invalid_argument", "src or dst is NULL");
        if (cols == 0) fail("invalid_launch", "quantized cols must be positive");
        lapid_b200_layout l = layout_of(format, rows, cols);
        uint64_t want = block_bytes(format) ? l.qs_bytes : rows * (cols / 32) * (format == LAPID_B200_DTYPE_INT4 ? 18 : 34);
        if (src_bytes != want || src->bytes < src_bytes)
            fail("shape_mismatch", "from_ggml_blocks: got " + std::to_string(src_bytes) + " bytes, expected " + std::to_string(want));
        if (dst->bytes < l.total)
            fail("out_of_bounds", "from_ggml_blocks: output holds " + std::to_string(dst->bytes) + " < " + std::to_string(l.total));
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        cuda_check(cudaMemsetAsync(dst->ptr, 0, l.total, dev->stream), "memset");
        if (block_bytes(format)) {
            if (want) cuda_check(cudaMemcpyAsync(dst->ptr, src->ptr, want, cudaMemcpyDeviceToDevice, dev->stream), "copy");
        } else if (format == LAPID_B200_DTYPE_INT4) {
            cuda_check(lb::launch_q4_0_to_planes(src->ptr, dst->ptr, l.scales_offset, rows * (cols / 32), dev->sm_count, dev->stream),
                       "q4_0 repack launch");
            dev->launches++;
        } else {
            cuda_check(lb::launch_q8_0_to_planes(src->ptr, dst->ptr, l.scales_offset, rows * (cols / 32), dev->sm_count, dev->stream),
                       "q8_0 repack launch");
            dev->launches++;
        }
        cuda_check(cudaStreamSynchronize(dev->stream), "from_ggml_blocks");
    });
}

uint64_t lapid_b200_tp_comm_bytes(int32_t world, uint64_t max_elems) {
    return world > 0 ? lb::tp_comm_bytes(world, max_elems) : 0;
}

lapid_b200_status lapid_b200_tp_comm_create(lapid_b200_device *dev, int32_t rank, int32_t world, void *const *peer_bases,
                                            uint64_t max_elems, lapid_b200_tp_comm **out) {
    return guard([&] {
        need(dev);
        if (!out || !peer_bases) fail("invalid_argument", "out or peer_bases is NULL");
        if (world < 1 || world > lb::TP_MAX_RANKS || rank < 0 || rank >= world)
            fail("invalid_argument", "tp: rank " + std::to_string(rank) + " of " + std::to_string(world) + " (at most " +
                                         std::to_string(lb::TP_MAX_RANKS) + " ranks)");
        if (max_elems == 0 || max_elems % 4) fail("invalid_argument", "tp: max_elems must be a positive multiple of 4");
        auto *c = new lapid_b200_tp_comm();
        for (int i = 0; i < world; i++) {
            if (!peer_bases[i] || ((uintptr_t)peer_bases[i] & 15)) {
                delete c;
                fail("invalid_argument", "tp: peer base " + std::to_string(i) + " is NULL or not 16-byte aligned");
            }
            c->args.peer[i] = peer_bases[i];
        }
        c->args.rank = rank;
        c->args.world = world;
        c->args.max_elems = max_elems;
        c->args.status = dev->status_dev;
        // the table the pushing kernels read, at the start of this rank's own buffer
        lb::TpPushTable table{};
        for (int i = 0; i < world; i++) table.peer[i] = peer_bases[i];
        table.max_elems = max_elems;
        table.rank = rank;
        table.world = world;
        {
            std::lock_guard<std::mutex> lock(dev->mu);
            dev->make_current();
            cudaError_t e = cudaMemcpy(peer_bases[rank], &table, sizeof(table), cudaMemcpyHostToDevice);
            if (e != cudaSuccess) {
                delete c;
                cuda_check(e, "cudaMemcpy(tp table)");
            }
        }
        dev->refs.fetch_add(1);
        c->dev = dev;
        *out = c;
    });
}

void lapid_b200_tp_comm_free(lapid_b200_tp_comm *comm) {
    if (!comm) return;
    device_release(comm->dev);
    delete comm;
}

lapid_b200_status lapid_b200_tp_all_reduce(lapid_b200_tp_comm *comm, lapid_b200_buffer *data, uint64_t offset, uint64_t count) {
    return guard([&] {
        if (!comm) fail("invalid_argument", "comm is NULL");
        need(data, "data");
        if (data->dev != comm->dev) fail("wrong_backend", "tp: data belongs to another device");
        if (count % 4 || count > comm->args.max_elems)
            fail("invalid_launch", "tp: count " + std::to_string(count) + " must be a multiple of 4 and <= " + std::to_string(comm->args.max_elems));
        if (offset % 4 || offset + count > data->bytes / 4)
            fail("out_of_bounds", "tp: [" + std::to_string(offset) + ", " + std::to_string(offset + count) + ") exceeds the buffer's " +
                                      std::to_string(data->bytes / 4) + " elements");
        lapid_b200_device *dev = comm->dev;
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        lb::TpAllReduceArgs a = comm->args;
        a.data = (float *)data->ptr + offset;
        a.count = count;
        a.spin_limit = dev->tp_spin_limit;
        cuda_check(lb::launch_tp_all_reduce(a, dev->pdl, dev->stream), "tp all-reduce launch");
        dev->launches++;
    });
}

// One decode MatMul launch whose result goes to the group: from the GEMV's own epilogue where the
// launch takes a K-quant fast kernel, else through its output buffer and a publishing kernel.
lapid_b200_status lapid_b200_tp_matmul_push(lapid_b200_tp_comm *comm, const lapid_b200_launch *launch,
                                            lapid_b200_buffer *const *buffers, size_t n_buffers) {
    return guard([&] {
        if (!comm) fail("invalid_argument", "comm is NULL");
        if (!launch) fail("invalid_argument", "launch is NULL");
        if (n_buffers && !buffers) fail("invalid_argument", "buffers is NULL");
        lapid_b200_device *dev = comm->dev;
        const lapid_b200_launch &l = *launch;
        const uint64_t count = l.batch * l.m * l.n;
        if (l.kind != LAPID_B200_KERNEL_MATMUL || l.batch * l.m > 8 || l.batch * l.m == 0)
            fail("invalid_launch", "tp push: a decode MatMul launch (1..8 rows) is required");
        if (count % 4 || count > comm->args.max_elems)
            fail("invalid_launch", "tp push: rows*n = " + std::to_string(count) + " must be a multiple of 4 and <= " + std::to_string(comm->args.max_elems));
        if (l.out.offset != 0 || l.out.row_stride != l.n || (l.batch > 1 && l.out.batch_stride != l.m * l.n))
            fail("invalid_launch", "tp push: the output view must be contiguous");
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        bool pushed = false;
        run_launch(*dev, l, buffers, n_buffers, nullptr, nullptr, (const lb::TpPushTable *)comm->args.peer[comm->args.rank], &pushed);
        if (!pushed) {
            lb::TpAllReduceArgs a = comm->args;
            a.data = (float *)buffers[l.output]->ptr;
            a.count = count;
            a.push_only = 1;
            cuda_check(lb::launch_tp_all_reduce(a, dev->pdl, dev->stream), "tp push launch");
            dev->launches++;
        }
    });
}

// rms_norm whose x is the sum of what the ranks pushed for the call in progress; closes the call.
lapid_b200_status lapid_b200_tp_rms_norm(lapid_b200_tp_comm *comm, lapid_b200_buffer *residual, lapid_b200_buffer *weight,
                                         lapid_b200_buffer *sum_out, lapid_b200_buffer *out, uint64_t rows, uint64_t cols, float eps) {
    return lapid_b200_tp_rms_norm_act(comm, residual, weight, sum_out, out, rows, cols, eps, nullptr, 0);
}

lapid_b200_status lapid_b200_tp_rms_norm_act(lapid_b200_tp_comm *comm, lapid_b200_buffer *residual, lapid_b200_buffer *weight,
                                             lapid_b200_buffer *sum_out, lapid_b200_buffer *out, uint64_t rows, uint64_t cols, float eps,
                                             lapid_b200_buffer *qact, int32_t layout) {
    return guard([&] {
        if (!comm) fail("invalid_argument", "comm is NULL");
        need(out, "out");
        lapid_b200_device *dev = comm->dev;
        if (rows == 0 || rows > 8 || !lb::rms_norm_shape_ok((uint32_t)(cols < (1ull << 31) ? cols : 0)) || rows * cols > comm->args.max_elems)
            fail("invalid_launch", "tp rms_norm: rows in 1..8, cols a multiple of 4 up to 16384, rows*cols <= " + std::to_string(comm->args.max_elems));
        const uint64_t bytes = rows * cols * 4;
        auto check = [&](lapid_b200_buffer *b, const char *what, uint64_t want) {
            if (!b) return;
            if (b->dev != dev) fail("wrong_backend", std::string("tp rms_norm: ") + what + " belongs to another device");
            if (b->bytes < want) fail("out_of_bounds", std::string("tp rms_norm ") + what + ": needs " + std::to_string(want) + " bytes, buffer has " + std::to_string(b->bytes));
            if ((uintptr_t)b->ptr & 15) fail("invalid_launch", std::string("tp rms_norm: ") + what + " must be 16-byte aligned");
        };
        check(residual, "residual", bytes);
        check(weight, "weight", cols * 4);
        check(sum_out, "sum_out", bytes);
        check(out, "out", bytes);
        if (out == residual || (sum_out && sum_out == out)) fail("buffer_aliasing", "tp rms_norm: out aliases residual or sum_out");
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        lb::RmsNormArgs a{};
        a.tp = (const lb::TpPushTable *)comm->args.peer[comm->args.rank];
        a.status = dev->status_dev;
        a.spin_limit = dev->tp_spin_limit;
        a.residual = residual ? (const float *)residual->ptr : nullptr;
        a.weight = weight ? (const float *)weight->ptr : nullptr;
        a.sum_out = sum_out ? (float *)sum_out->ptr : nullptr;
        a.out = (float *)out->ptr;
        a.rows = (uint32_t)rows;
        a.cols = (uint32_t)cols;
        a.eps = eps;
        a.q = act_out_checked(dev, qact, layout, rows, cols, "tp rms_norm");
        if (qact && !lb::rms_norm_quant_ok((uint32_t)cols)) fail("invalid_launch", "tp rms_norm: cols " + std::to_string(cols) + " cannot be quantized in the kernel");
        cuda_check(lb::launch_rms_norm(a, dev->pdl, dev->stream), "tp rms_norm launch");
        dev->launches++;
    });
}

// ---- the steps between projections (glue.cu); queued on the device's stream, not waited for
lapid_b200_status lapid_b200_rms_norm(lapid_b200_device *dev, lapid_b200_buffer *x, lapid_b200_buffer *residual,
                                      lapid_b200_buffer *weight, lapid_b200_buffer *sum_out, lapid_b200_buffer *out,
                                      uint64_t rows, uint64_t cols, float eps) {
    return lapid_b200_rms_norm_act(dev, x, residual, weight, sum_out, out, rows, cols, eps, nullptr, 0);
}

lapid_b200_status lapid_b200_rms_norm_act(lapid_b200_device *dev, lapid_b200_buffer *x, lapid_b200_buffer *residual,
                                          lapid_b200_buffer *weight, lapid_b200_buffer *sum_out, lapid_b200_buffer *out,
                                          uint64_t rows, uint64_t cols, float eps, lapid_b200_buffer *qact, int32_t layout) {
    return guard([&] {
        need(dev);
        need(x, "x");
        need(out, "out");
        if (rows >= (1ull << 31) || !lb::rms_norm_shape_ok((uint32_t)(cols < (1ull << 31) ? cols : 0)))
            fail("invalid_launch", "rms_norm: cols must be a multiple of 4 in 4..16384, got " + std::to_string(cols));
        const uint64_t bytes = rows * cols * 4;
        auto check = [&](lapid_b200_buffer *b, const char *what, uint64_t want) {
            if (!b) return;
            if (b->dev != dev) fail("wrong_backend", std::string("rms_norm: ") + what + " belongs to another device");
            if (b->bytes < want) fail("out_of_bounds", std::string("rms_norm ") + what + ": needs " + std::to_string(want) + " bytes, buffer has " + std::to_string(b->bytes));
            if ((uintptr_t)b->ptr & 15) fail("invalid_launch", std::string("rms_norm: ") + what + " must be 16-byte aligned");
        };
        check(x, "x", bytes);
        check(residual, "residual", bytes);
        check(weight, "weight", cols * 4);
        check(sum_out, "sum_out", bytes);
        check(out, "out", bytes);
        if (out == x || out == residual || (sum_out && sum_out == out)) fail("buffer_aliasing", "rms_norm: out aliases an input or sum_out");
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        lb::RmsNormArgs a{};
        a.x = (const float *)x->ptr;
        a.residual = residual ? (const float *)residual->ptr : nullptr;
        a.weight = weight ? (const float *)weight->ptr : nullptr;
        a.sum_out = sum_out ? (float *)sum_out->ptr : nullptr;
        a.out = (float *)out->ptr;
        a.rows = (uint32_t)rows;
        a.cols = (uint32_t)cols;
        a.eps = eps;
        a.q = act_out_checked(dev, qact, layout, rows, cols, "rms_norm");
        if (qact && !lb::rms_norm_quant_ok((uint32_t)cols)) fail("invalid_launch", "rms_norm: cols " + std::to_string(cols) + " cannot be quantized in the kernel");
        cuda_check(lb::launch_rms_norm(a, dev->pdl, dev->stream), "rms_norm launch");
        dev->launches++;
    });
}

lapid_b200_status lapid_b200_silu_mul(lapid_b200_device *dev, lapid_b200_buffer *gate, lapid_b200_buffer *up,
                                      lapid_b200_buffer *out, uint64_t count) {
    return lapid_b200_silu_mul_act(dev, gate, up, out, 1, count, nullptr, 0);
}

lapid_b200_status lapid_b200_act_layout(lapid_b200_device *dev, const lapid_b200_launch *launch, int32_t *layout, uint64_t *bytes) {
    return guard([&] {
        need(dev);
        if (!launch || !layout || !bytes) fail("invalid_argument", "launch, layout or bytes is NULL");
        if (launch->kind != LAPID_B200_KERNEL_MATMUL) fail("invalid_launch", "act_layout: not a MatMul launch");
        Plan p = plan_launch(*dev, *launch);
        if (!p.gemv || p.noop || p.zero_k || launch->k % 256 != 0)
            fail("invalid_launch", "act_layout: the launch does not take a quantized activation operand (batch*m <= " +
                                       std::to_string(dev->gemv_max_rows) + ", k a multiple of 256)");
        *layout = p.records();
        *bytes = p.scratch;
    });
}

// The pre-pass of the decode path as a call of its own (crates/lapid-cpu/src/matmul/quant.rs:30-89).
lapid_b200_status lapid_b200_quantize_activations(lapid_b200_device *dev, const lapid_b200_buffer *a, uint64_t rows, uint64_t k,
                                                  int32_t layout, lapid_b200_buffer *qact) {
    return guard([&] {
        need(dev);
        if (!a || !qact) fail("invalid_argument", "a or qact is NULL");
        if (a->dev != dev || qact->dev != dev) fail("wrong_backend", "quantize_activations: a buffer belongs to another device");
        if (rows == 0 || rows > 8 || k == 0 || k >= (1ull << 31) || k % 32 != 0 || (layout != 0 && k % 256 != 0))
            fail("invalid_launch", "quantize_activations: rows in 1..8, k a multiple of 32 (of 256 for the record and tile layouts)");
        if (layout < 0 || layout > 2) fail("invalid_argument", "quantize_activations: layout must be 0, 1 or 2");
        if (a->bytes / 4 < rows * k) fail("out_of_bounds", "quantize_activations: a holds " + std::to_string(a->bytes / 4) + " < " + std::to_string(rows * k) + " elements");
        if ((uintptr_t)a->ptr & 15) fail("invalid_launch", "quantize_activations: a must be 16-byte aligned");
        const size_t planes = lb::act_plane_bytes((uint32_t)rows, (uint32_t)k) + 2 * lb::act_scale_bytes((uint32_t)rows, (uint32_t)k);
        const size_t need_b = layout == 0 ? planes : layout == 1 ? rows * (k / 256) * lb::REC : lb::qgemv_q4k_mma_act_bytes((uint32_t)rows, (uint32_t)k);
        if (qact->bytes < need_b) fail("out_of_bounds", "quantize_activations qact: needs " + std::to_string(need_b) + " bytes, buffer has " + std::to_string(qact->bytes));
        if ((uintptr_t)qact->ptr & 15) fail("invalid_launch", "quantize_activations: qact must be 16-byte aligned");
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        const lb::ActOut o = act_out_at(qact->ptr, layout, (uint32_t)rows, (uint32_t)k);
        lb::ActQuantArgs q{};
        q.a = a->ptr;
        q.a_bs = rows * k;
        q.a_rs = k;
        q.rows = (uint32_t)rows;
        q.m = (uint32_t)rows;
        q.k = (uint32_t)k;
        q.qa = o.qa;
        q.da = o.da;
        q.bs = o.bs;
        q.records = layout;
        cuda_check(lb::launch_act_quant(q, dev->sm_count, dev->pdl, dev->stream), "act_quant launch");
        dev->launches++;
    });
}

lapid_b200_status lapid_b200_silu_mul_act(lapid_b200_device *dev, lapid_b200_buffer *gate, lapid_b200_buffer *up,
                                          lapid_b200_buffer *out, uint64_t rows, uint64_t cols, lapid_b200_buffer *qact, int32_t layout) {
    const uint64_t count = rows * cols;
    return guard([&] {
        need(dev);
        need(gate, "gate");
        need(up, "up");
        need(out, "out");
        if (count % 4) fail("invalid_launch", "silu_mul: count must be a multiple of 4, got " + std::to_string(count));
        for (lapid_b200_buffer *b : {gate, up, out}) {
            if (b->dev != dev) fail("wrong_backend", "silu_mul: a buffer belongs to another device");
            if (b->bytes < count * 4) fail("out_of_bounds", "silu_mul: needs " + std::to_string(count * 4) + " bytes, a buffer has " + std::to_string(b->bytes));
            if ((uintptr_t)b->ptr & 15) fail("invalid_launch", "silu_mul: buffers must be 16-byte aligned");
        }
        std::lock_guard<std::mutex> lock(dev->mu);
        dev->make_current();
        lb::ActOut q = act_out_checked(dev, qact, layout, rows, cols, "silu_mul");
        cuda_check(lb::launch_silu_mul((const float *)gate->ptr, (const float *)up->ptr, (float *)out->ptr, count, (uint32_t)(qact ? cols : 0), q,
                                       dev->sm_count, dev->pdl, dev->stream), "silu_mul launch");
        dev->launches++;
    });
}

}  // extern "C"

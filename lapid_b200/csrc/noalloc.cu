// lapid_b200_gemv_q4k_static: the Q4_K decode GEMV for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the time they need a matvec: an engine that
// hands every byte of device memory to its own arena at start-up, a serving loop that has promised
// a fixed memory footprint, a plug-in that runs under another runtime's allocator and may not touch
// the CUDA one. The regular entry points keep the quantized activations in a scratch block that the
// device object grows with cudaMalloc; this entry point keeps them in an array that is part of the
// library image instead, so the only memory it touches besides the caller's inputs and outputs was
// reserved when the library was loaded.
//
// Consequences the caller has to know:
//  * the array is LAPID_B200_STATIC_SCRATCH_BYTES (84 KiB) and every GPU that loads the library
//    carries it until the process exits; rows * k is therefore limited (see the header);
//  * there is one array per GPU and every call on that GPU uses it: two calls that may overlap on
//    the GPU (different streams, no event between them) race on it. Calls on one stream are safe;
//  * the array keeps what the last call left in it. Nothing in it has to start at zero: the
//    pre-pass of a call overwrites every byte its GEMV interprets (the 16 padding bytes of a
//    record are copied but never read as data);
//  * the first call on a GPU looks up the array's device address; the first call on a GPU with a given
//    (rows, k) also sets that kernel variant's attributes and asks for its occupancy. Make those first
//    calls outside any stream capture; later calls with the same shape only launch two kernels;
//  * the calling thread's current device is `ordinal` while the call runs and is put back before it returns;
//  * a device-side wait that gives up (it never should) is recorded in a second static word, which
//    lapid_b200_gemv_q4k_static_status reads and clears.
// No cudaMalloc, cudaFree, cudaHostAlloc or any other allocating call is made here, on any path.
#include "../../include/lapid_b200.h"

#include <mutex>
#include <string>

#include "common.cuh"
#include "kernels.h"

namespace lb {
int32_t report_error(const char *code, const std::string &message);  // backend.cc: status + last-error JSON
}

namespace {

constexpr size_t STATIC_SCRATCH_BYTES = LAPID_B200_STATIC_SCRATCH_BYTES;

// Activation records of one call: rows * (k / 256) records of 336 bytes. In host code this name is
// only a handle for cudaGetSymbolAddress; the kernels get the looked-up device address.
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];
// The kernels OR a bit in here when one of their bounded waits gave up (the role the host-mapped status word
// of a device object plays for `execute`).
static __device__ int g_static_status;

constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
void *g_scratch_addr[MAX_DEVICES] = {};
int *g_status_addr[MAX_DEVICES] = {};
int g_sm_count[MAX_DEVICES] = {};

// Makes `ordinal` current for the scope and puts the caller's device back afterwards.
struct DeviceScope {
    int prev = -1;
    cudaError_t err;
    explicit DeviceScope(int ordinal) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        err = cudaSetDevice(ordinal);
    }
    ~DeviceScope() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

}  // namespace

extern "C" LAPID_B200_API lapid_b200_status lapid_b200_gemv_q4k_static(int32_t ordinal, void *cuda_stream, const float *a,
                                                                       const void *w, uint64_t w_bytes, float *out,
                                                                       uint32_t rows, uint32_t n, uint32_t k) {
    if (!a || !w || !out) return lb::report_error("invalid_argument", "gemv_q4k_static: a, w or out is NULL");
    if (ordinal < 0 || ordinal >= MAX_DEVICES)
        return lb::report_error("device_unavailable", "gemv_q4k_static: device ordinal " + std::to_string(ordinal));
    if (rows < 1 || rows > 8) return lb::report_error("invalid_launch", "gemv_q4k_static: rows must be in 1..8, got " + std::to_string(rows));
    if (k == 0 || k % lb::QK != 0)
        return lb::report_error("invalid_launch", "gemv_q4k_static: k must be a positive multiple of 256, got " + std::to_string(k));
    if (n == 0) return LAPID_B200_OK;
    const uint64_t need = (uint64_t)rows * (k / lb::QK) * lb::REC;
    if (need > STATIC_SCRATCH_BYTES)
        return lb::report_error("too_large", "gemv_q4k_static: rows * k / 256 = " + std::to_string((uint64_t)rows * (k / lb::QK)) +
                                                 " activation records need " + std::to_string(need) + " bytes, the static scratch holds " +
                                                 std::to_string(STATIC_SCRATCH_BYTES) + " (rows * k <= 65536)");
    const uint64_t w_need = (uint64_t)n * (k / lb::QK) * lb::Q4K_BYTES;
    if (w_bytes < w_need)
        return lb::report_error("out_of_bounds", "gemv_q4k_static: quantized [" + std::to_string(n) + ", " + std::to_string(k) + "] needs " +
                                                     std::to_string(w_need) + " bytes, got " + std::to_string(w_bytes));
    if (((uintptr_t)w & 15) != 0) return lb::report_error("invalid_launch", "gemv_q4k_static: w must be 16-byte aligned");

    DeviceScope scope(ordinal);
    cudaError_t e = scope.err;
    if (e != cudaSuccess) return lb::report_error("device_unavailable", std::string("gemv_q4k_static: cudaSetDevice: ") + cudaGetErrorString(e));
    void *scratch = nullptr;
    int *status = nullptr;
    int sm_count = 0;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_scratch_addr[ordinal]) {  // set-up, once per device, with that device current
            void *ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_static_scratch);
            if (e != cudaSuccess || !ptr)
                return lb::report_error("cuda", std::string("gemv_q4k_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
            void *sptr = nullptr;
            e = cudaGetSymbolAddress(&sptr, g_static_status);
            if (e != cudaSuccess || !sptr)
                return lb::report_error("cuda", std::string("gemv_q4k_static: cudaGetSymbolAddress(status): ") + cudaGetErrorString(e));
            int sms = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ordinal);
            if (e != cudaSuccess) return lb::report_error("cuda", std::string("gemv_q4k_static: ") + cudaGetErrorString(e));
            g_sm_count[ordinal] = sms;
            g_status_addr[ordinal] = (int *)sptr;
            g_scratch_addr[ordinal] = ptr;
        }
        scratch = g_scratch_addr[ordinal];
        status = g_status_addr[ordinal];
        sm_count = g_sm_count[ordinal];
    }
    cudaStream_t stream = (cudaStream_t)cuda_stream;

    lb::ActQuantArgs q{};
    q.a = a;
    q.a_off = 0;
    q.a_bs = 0;
    q.a_rs = k;
    q.rows = rows;
    q.m = rows;
    q.k = k;
    q.qa = (int8_t *)scratch;
    q.da = nullptr;
    q.bs = nullptr;
    q.records = 1;
    e = lb::launch_act_quant(q, sm_count, false, stream);
    if (e != cudaSuccess) return lb::report_error("cuda", std::string("gemv_q4k_static: pre-pass launch: ") + cudaGetErrorString(e));

    lb::GemvArgs g{};
    g.w = (const uint8_t *)w;
    g.w_bytes = w_bytes;
    g.qa = (const int8_t *)scratch;
    g.out = out;
    g.out_off = 0;
    g.out_bs = 0;
    g.out_rs = n;
    g.extra = nullptr;
    g.a = a;
    g.a_rs = k;
    g.status = status;
    g.rows = rows;
    g.m = rows;
    g.n = n;
    g.k = k;
    if (!lb::qgemv_q4k_fast_supported(g)) return lb::report_error("invalid_launch", "gemv_q4k_static: shape not supported");
    e = lb::launch_qgemv_q4k_fast(g, sm_count, false, stream);
    if (e != cudaSuccess) return lb::report_error("cuda", std::string("gemv_q4k_static: launch: ") + cudaGetErrorString(e));
    return LAPID_B200_OK;
}

// Reads and clears the wait-timeout word of `ordinal`'s static path. Synchronise the stream(s) the calls were
// queued on first: the copy below is ordered behind the legacy default stream only.
extern "C" LAPID_B200_API lapid_b200_status lapid_b200_gemv_q4k_static_status(int32_t ordinal, int32_t *out) {
    if (!out) return lb::report_error("invalid_argument", "gemv_q4k_static_status: out is NULL");
    if (ordinal < 0 || ordinal >= MAX_DEVICES)
        return lb::report_error("device_unavailable", "gemv_q4k_static_status: device ordinal " + std::to_string(ordinal));
    int *addr = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        addr = g_status_addr[ordinal];
    }
    if (!addr) {  // no call on this GPU yet: nothing can have been recorded
        *out = 0;
        return LAPID_B200_OK;
    }
    DeviceScope scope(ordinal);
    if (scope.err != cudaSuccess)
        return lb::report_error("device_unavailable", std::string("gemv_q4k_static_status: cudaSetDevice: ") + cudaGetErrorString(scope.err));
    int v = 0;
    cudaError_t e = cudaMemcpy(&v, addr, sizeof v, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && v != 0) e = cudaMemset(addr, 0, sizeof v);
    if (e != cudaSuccess) return lb::report_error("cuda", std::string("gemv_q4k_static_status: ") + cudaGetErrorString(e));
    *out = v;
    return LAPID_B200_OK;
}

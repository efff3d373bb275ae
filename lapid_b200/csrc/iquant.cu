// The i-quant codebooks on the device (see iquant.cuh). The 15488 bytes come from the file iq_grids.bin beside this
// source, which the build embeds into the library; one copy per device is uploaded when a device handle is
// created.
#include <mutex>

#include "iquant.cuh"

#ifndef LAPID_B200_IQ_GRIDS_FILE
#error "LAPID_B200_IQ_GRIDS_FILE must name iq_grids.bin"
#endif
#define LB_STR2(x) #x
#define LB_STR(x) LB_STR2(x)
__asm__(".section .rodata\n"
        ".balign 16\n"
        "lapid_b200_iq_grids_blob:\n"
        ".incbin \"" LB_STR(LAPID_B200_IQ_GRIDS_FILE) "\"\n"
        "lapid_b200_iq_grids_blob_end:\n"
        ".previous\n");
extern "C" const unsigned char lapid_b200_iq_grids_blob[] __attribute__((visibility("hidden")));
extern "C" const unsigned char lapid_b200_iq_grids_blob_end[] __attribute__((visibility("hidden")));

namespace lb {

namespace {
constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
uint8_t *g_table[MAX_DEVICES] = {};
}  // namespace

const uint8_t *iq_grids() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
    std::lock_guard<std::mutex> lock(g_mu);
    return g_table[dev];
}

cudaError_t iq_grids_upload() {
    if (lapid_b200_iq_grids_blob_end - lapid_b200_iq_grids_blob != IQ_GRID_BYTES) return cudaErrorInvalidValue;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= MAX_DEVICES) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_table[dev]) return cudaSuccess;
    uint8_t *p = nullptr;
    if ((e = cudaMalloc(&p, IQ_GRID_BYTES)) != cudaSuccess) return e;
    if ((e = cudaMemcpy(p, lapid_b200_iq_grids_blob, IQ_GRID_BYTES, cudaMemcpyHostToDevice)) != cudaSuccess) {
        cudaFree(p);
        return e;
    }
    g_table[dev] = p;
    return cudaSuccess;
}

}  // namespace lb

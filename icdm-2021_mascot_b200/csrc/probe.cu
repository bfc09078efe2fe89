// Measurement utility of the library (no counterpart in the reference): how fast the SMs of a device
// read a buffer with 128-bit L2-only loads - the access the update kernel makes for every factor row.
// A buffer that fits in L2 gives the L2 -> SM bandwidth against which the update kernel's L2 traffic is
// judged when the factors are L2-resident; a buffer far larger than L2 gives the HBM read bandwidth.
#include <cuda_runtime.h>

#include "handle.h"

namespace mascot {
namespace {

__global__ void __launch_bounds__(256) read_probe_kernel(const uint4* buf, size_t n16, unsigned passes, unsigned* sink) {
    unsigned acc = 0;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (unsigned p = 0; p < passes; p++)
        for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < n16; j += stride) {
            const uint4 v = __ldcg(buf + j);
            acc ^= v.x ^ v.y ^ v.z ^ v.w;
        }
    if (acc == 0x9e3779b9u) *sink = acc;          // keeps the loads alive; practically never taken
}

}  // namespace
}  // namespace mascot

using namespace mascot;

extern "C" int mascot_probe_read_bandwidth(int device, uint64_t bytes, uint32_t passes, double* gb_per_s) {
    if (!gb_per_s || bytes < 4096 || !passes) return fail(nullptr, MASCOT_ERR_BAD_ARG, "bad probe arguments");
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev) {
        cudaGetLastError();
        return fail(nullptr, MASCOT_ERR_NO_DEVICE, "no usable CUDA device");
    }
    CU(nullptr, cudaSetDevice(device));
    const size_t n16 = bytes / 16;
    uint4* buf = nullptr; unsigned* sink = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaError_t e = cudaMalloc(&buf, n16 * 16);
    if (e == cudaSuccess) e = cudaMalloc(&sink, sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemset(buf, 1, n16 * 16);
    if (e == cudaSuccess) e = cudaEventCreate(&e0);
    if (e == cudaSuccess) e = cudaEventCreate(&e1);
    float ms = 0.f;
    if (e == cudaSuccess) {
        const int grid = sm_count() * 8;
        read_probe_kernel<<<grid, 256>>>(buf, n16, 1, sink);              // warm-up pass (fills L2 when the buffer fits)
        cudaEventRecord(e0);
        read_probe_kernel<<<grid, 256>>>(buf, n16, passes, sink);
        cudaEventRecord(e1);
        e = cudaEventSynchronize(e1);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(buf); cudaFree(sink);
    CU(nullptr, e);
    *gb_per_s = ms > 0.f ? (double)(n16 * 16) * passes / (ms * 1e-3) / 1e9 : 0.0;
    return MASCOT_OK;
}

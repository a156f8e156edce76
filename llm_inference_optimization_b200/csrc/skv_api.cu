// Library-wide C-ABI entry points that belong to no single kernel.
#include "skv_common.cuh"

extern "C" {

// Message for the most recent non-zero status returned on the calling thread.
const char* skv_last_error(void) { return skv::last_error_buf(); }

// ABI revision; bumped whenever a signature in include/skv_b200.h changes.
int skv_abi_version(void) { return 2; }

// Reads the device status word at offset 0 of a workspace (bit SKV_DEV_TIMEOUT set
// when a bounded wait inside a kernel gave up).  Synchronises `stream`.
int skv_workspace_status(const void* workspace, int device, void* stream, int* status_out) {
    if (!workspace || !status_out) return skv::fail(SKV_ERR_BAD_ARG, "skv_workspace_status: null pointer");
    skv::DeviceGuard guard(device);
    if (!guard.ok) return skv::fail(SKV_ERR_CUDA, "cannot switch to device %d", device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    SKV_CUDA_TRY(cudaMemcpyAsync(status_out, workspace, sizeof(int),
                                 cudaMemcpyDeviceToHost, st));
    SKV_CUDA_TRY(cudaStreamSynchronize(st));
    return SKV_OK;
}

}  // extern "C"

#ifdef SKV_BOUNDS
// Self-test of the range-check instrumentation: a kernel pushes one index that is in range and one that is not
// through SKV_INDEX without touching memory through them; returns what the macro gave back and what it recorded.
namespace skv {
__global__ void bounds_selftest_kernel(int* out) {
    const int i = threadIdx.x;           // not a compile-time constant
    out[0] = SKV_INDEX(i + 2, 3);        // in range: 2
    out[1] = SKV_INDEX(i + 5, 3);        // out of range: replaced by 0, line recorded
}
}  // namespace skv
extern "C" int skv_debug_bounds_selftest(int* in_range, int* clamped, int* recorded_line) {
    int* d = nullptr;
    int h[2] = {-1, -1};
    if (cudaMalloc(&d, 2 * sizeof(int)) != cudaSuccess) return SKV_ERR_CUDA;
    skv::bounds_selftest_kernel<<<1, 1>>>(d);
    cudaError_t e = cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
    cudaFree(d);
    if (e != cudaSuccess) return SKV_ERR_CUDA;
    *in_range = h[0];
    *clamped = h[1];
    return cudaMemcpyFromSymbol(recorded_line, skv::skv_bounds_word, sizeof(int)) == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}
#endif

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

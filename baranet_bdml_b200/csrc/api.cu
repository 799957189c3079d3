// Status/error plumbing of the C ABI (include/bn_attn.h).
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace bn {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int require_sm100() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(BN_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    static thread_local int cached_dev = -1;
    static thread_local int cached_major = 0;
    if (dev != cached_dev) {
        int major = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) return fail(BN_ERR_CUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
        cached_dev = dev;
        cached_major = major;
    }
    if (cached_major != 10)
        return fail(BN_ERR_ARCH, "device %d has compute capability %d.x; this library is built for sm_100a only",
                    dev, cached_major);
    return BN_OK;
}

int launch_status(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(BN_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return BN_OK;
}

}  // namespace bn

extern "C" {

const char* bn_last_error(void) { return bn::g_err; }

int bn_version(void) { return 100; }

int bn_workspace_status(const void* workspace, bn_stream_t stream) {
    if (!workspace) return bn::fail(BN_ERR_INVALID_ARG, "bn_workspace_status: null workspace");
    int word = 0;   // every scratch layout keeps its error word first
    cudaError_t e = cudaMemcpyAsync(&word, workspace, sizeof(word), cudaMemcpyDeviceToHost, bn::as_stream(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(bn::as_stream(stream));
    if (e != cudaSuccess) return bn::fail(BN_ERR_CUDA, "bn_workspace_status: %s", cudaGetErrorString(e));
    if (word == BN_ERR_TIMEOUT)
        return bn::fail(BN_ERR_TIMEOUT, "a bounded device-side wait ran out; the result is invalid");
    return BN_OK;
}

}  // extern "C"

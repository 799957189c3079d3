// Status/error plumbing of the C ABI (include/bn_attn.h).
#include <cstdarg>
#include <cstdio>

#include "common.cuh"
#include "ptx.cuh"

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

// The bounded wait of every kernel here (ptx::mbar_wait), on a barrier that nothing ever arrives at: the wait gives
// up after `limit_ns`, raises the CTA's abort flag, and the kernel stores BN_ERR_TIMEOUT in the error word at the
// head of the scratch buffer and returns - the path a kernel takes when a producer never delivers.
__global__ void wait_that_runs_out_kernel(int* error_word, unsigned long long limit_ns) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int s_abort;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        s_abort = 0;
        ptx::fence_mbar_init();
    }
    __syncthreads();
    // every warp waits; the first one whose limit expires raises the flag, the others leave on seeing it
    const bool ok = ptx::mbar_wait(ptx::smem_u32(&bar), 0, &s_abort, limit_ns);
    __syncthreads();
    if (threadIdx.x == 0 && (!ok || s_abort)) atomicExch(error_word, BN_ERR_TIMEOUT);
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

int bn_selftest_wait_timeout(void* workspace, unsigned limit_us, bn_stream_t stream) {
    if (!workspace) return bn::fail(BN_ERR_INVALID_ARG, "bn_selftest_wait_timeout: null workspace");
    if (limit_us == 0 || limit_us > 100000) return bn::fail(BN_ERR_INVALID_ARG, "bn_selftest_wait_timeout: limit of 1..100000 us");
    if (int rc = bn::require_sm100()) return rc;
    bn::wait_that_runs_out_kernel<<<2, 128, 0, bn::as_stream(stream)>>>(static_cast<int*>(workspace),
                                                                        (unsigned long long)limit_us * 1000ull);
    return bn::launch_status("bn_selftest_wait_timeout");
}

}  // extern "C"

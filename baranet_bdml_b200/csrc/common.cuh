// Shared helpers of the attention module: status/error plumbing and small
// device utilities.  Everything here is internal; the public surface is
// include/bn_attn.h.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "bn_attn.h"

namespace bn {

// Records `code` and a printf-style message for bn_last_error(); returns code.
int fail(int code, const char* fmt, ...);

// BN_OK when the current device is compute capability 10.x, else BN_ERR_ARCH.
int require_sm100();

// Converts a pending launch error into BN_ERR_CUDA.
int launch_status(const char* what);

inline cudaStream_t as_stream(bn_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Launches `kernel` as a programmatic dependent of the stream's previous kernel: it may be scheduled while that
// kernel is still running, so the kernel must execute griddepcontrol.wait before its first access to global memory
// that depends on earlier work (everything but constant weights).  What this buys is the launch latency and the
// kernel's own prologue, hidden under the predecessor's tail - the decode step is a chain of ~180 short kernels.
// Falls back to an ordinary launch if the attribute is refused.
template <typename... P, typename... A>
inline void launch_dependent(void (*kernel)(P...), unsigned grid, unsigned block, size_t smem, cudaStream_t st, A... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, args...) != cudaSuccess) {
        (void)cudaGetLastError();
        kernel<<<grid, block, smem, st>>>(args...);
    }
}

// Byte offsets inside the scratch buffer of bn_attn_prefill_bf16 (cos/sin table, per-tile key norms, rotated K) and
// its size: the fused q/k/v projection writes the last two itself.
void prefill_bf16_workspace_layout(int B, int S, int Hkv, size_t* table, size_t* kmax2, size_t* krot, size_t* total);

// The RoPE frequency of pair i, with the reference's exact arithmetic
// (src/ops/op_rope.cuh:82): fp32 exponent, fp32 pow, reciprocal taken in
// double, rounded to fp32.
__device__ __forceinline__ float rope_inv_freq(int pair, int head_dim, float theta) {
    return (float)(1.0 / powf(theta, (float)(2 * pair) / head_dim));
}

}  // namespace bn

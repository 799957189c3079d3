// RMSNorm and residual-add + RMSNorm, fp32, bit-compatible with the reference operator.
//
//   bn_rmsnorm_f32      y = x / sqrt(mean(x^2) + eps) * w, row-wise
//                       reference: op_rmsnorm (src/ops/op_rmsnorm.cuh:8-53, launcher :134-157)
//   bn_add_rmsnorm_f32  s = a + b;  y = rmsnorm(s)  in one pass over the row: the decoder layer's
//                       `residual + hidden_states` (op_add) followed by the next layer norm
//                       (mygrad/llama/llama_layers.py:279-283), which the reference runs as two launches with the
//                       sum written and read back in between
//
// The reference kernel's arithmetic order is part of its result, so it is kept: 256 threads per row, thread t owns
// elements t, t + 256, ... and accumulates their squares as ONE fused-multiply-add chain in that order; the 256
// partial sums are reduced by the tree  sh[t] += sh[t + stride], stride = 128 ... 1;  mean = total / hidden and
// x / rms are IEEE divisions, rms an IEEE square root.  (The tree's last five levels run as warp shuffles: lane t
// adds lane t + stride, the same pairs in the same order.)
//
// HBM-bound: a row is read once (its elements stay in registers between the two passes when hidden <= 4096) and
// written once; 4 bytes per thread and access, consecutive threads on consecutive elements, so every warp access
// is one full 128-byte line; 8 rows (CTAs) per SM keep about 64 KB in flight per SM.
#include "common.cuh"

namespace bn {

constexpr int RN_THREADS = 256;      // fixed by the reference's reduction layout
constexpr int RN_MAXV = 16;          // most elements per thread kept in registers (hidden <= 4096)

struct RmsParams {
    const float* a; int64_t a_rs, a_cs;
    const float* b; int64_t b_rs, b_cs;     // optional residual (nullptr: none)
    const float* w; int64_t w_cs;
    float* s; int64_t s_rs, s_cs;           // optional: the sum a + b
    float* y; int64_t y_rs, y_cs;
    int rows, hidden;
    float eps;
};

// Reduction of the 256 partial sums in the reference's tree order, then rms = sqrt(total / hidden + eps).
// Strides 128 and 64 go through shared memory, 32 by warp 0 from shared memory, 16..1 as shuffles (lane t adds lane
// t + stride: the same pairs).  All threads return the row's rms.
__device__ __forceinline__ float row_rms(float acc, float* sh, float* s_rms, int hidden, float eps) {
    const int tid = threadIdx.x;
    sh[tid] = acc;
    __syncthreads();
    if (tid < 128) sh[tid] = __fadd_rn(sh[tid], sh[tid + 128]);
    __syncthreads();
    if (tid < 64) sh[tid] = __fadd_rn(sh[tid], sh[tid + 64]);
    __syncthreads();
    if (tid < 32) {
        float t = __fadd_rn(sh[tid], sh[tid + 32]);
#pragma unroll
        for (int stride = 16; stride > 0; stride >>= 1) t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, stride));
        if (tid == 0) *s_rms = __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)hidden), eps));
    }
    __syncthreads();
    return *s_rms;     // sh / s_rms are rewritten only after the next row's first barrier
}

// NV = elements per thread held in registers between the two passes (hidden <= 256 NV).  The loads of the CTA's
// NEXT row are issued before the reduction of the current one, so memory requests stay in flight across the
// barriers of the reduction.
template <int NV, bool ADD>
__global__ void __launch_bounds__(RN_THREADS, NV == 16 ? 2 : 4)
rmsnorm_regs_kernel(const RmsParams p) {
    __shared__ float sh[RN_THREADS];
    __shared__ float s_rms;
    const int tid = threadIdx.x;
    float v[NV], na[NV], nb[ADD ? NV : 1];
    auto load_row = [&](int row) {
        const float* ar = p.a + (int64_t)row * p.a_rs;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int i = tid + k * RN_THREADS;
            na[k] = i < p.hidden ? __ldg(ar + (int64_t)i * p.a_cs) : 0.f;
        }
        if (ADD) {
            const float* br = p.b + (int64_t)row * p.b_rs;
#pragma unroll
            for (int k = 0; k < NV; ++k) {
                const int i = tid + k * RN_THREADS;
                nb[ADD ? k : 0] = i < p.hidden ? __ldg(br + (int64_t)i * p.b_cs) : 0.f;
            }
        }
    };
    int row = blockIdx.x;
    if (row < p.rows) load_row(row);
    for (; row < p.rows; row += gridDim.x) {
#pragma unroll
        for (int k = 0; k < NV; ++k) v[k] = ADD ? __fadd_rn(na[k], nb[ADD ? k : 0]) : na[k];
        if (row + (int)gridDim.x < p.rows) load_row(row + gridDim.x);
        // the chain in the reference's order
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < NV; ++k)
            if (tid + k * RN_THREADS < p.hidden) acc = __fmaf_rn(v[k], v[k], acc);
        const float rms = row_rms(acc, sh, &s_rms, p.hidden, p.eps);
        float* sr = p.s ? p.s + (int64_t)row * p.s_rs : nullptr;
        float* yr = p.y + (int64_t)row * p.y_rs;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int i = tid + k * RN_THREADS;
            if (i < p.hidden) {
                if (ADD && sr) sr[(int64_t)i * p.s_cs] = v[k];
                yr[(int64_t)i * p.y_cs] = __fmul_rn(__fdiv_rn(v[k], rms), __ldg(p.w + (int64_t)i * p.w_cs));
            }
        }
    }
}

// any width: the row is read twice (the second read hits L2)
__global__ void __launch_bounds__(RN_THREADS)
rmsnorm_wide_kernel(const RmsParams p) {
    __shared__ float sh[RN_THREADS];
    __shared__ float s_rms;
    const int tid = threadIdx.x;
    for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const float* ar = p.a + (int64_t)row * p.a_rs;
        const float* br = p.b ? p.b + (int64_t)row * p.b_rs : nullptr;
        float* sr = p.s ? p.s + (int64_t)row * p.s_rs : nullptr;
        float* yr = p.y + (int64_t)row * p.y_rs;
        float acc = 0.f;
        for (int i = tid; i < p.hidden; i += RN_THREADS) {
            float x = __ldg(ar + (int64_t)i * p.a_cs);
            if (br) x = __fadd_rn(x, __ldg(br + (int64_t)i * p.b_cs));
            acc = __fmaf_rn(x, x, acc);
        }
        const float rms = row_rms(acc, sh, &s_rms, p.hidden, p.eps);
        for (int i = tid; i < p.hidden; i += RN_THREADS) {
            float x = __ldg(ar + (int64_t)i * p.a_cs);
            if (br) x = __fadd_rn(x, __ldg(br + (int64_t)i * p.b_cs));
            if (sr) sr[(int64_t)i * p.s_cs] = x;
            yr[(int64_t)i * p.y_cs] = __fmul_rn(__fdiv_rn(x, rms), __ldg(p.w + (int64_t)i * p.w_cs));
        }
    }
}

static int rmsnorm_launch(const RmsParams& p, bn_stream_t stream, const char* what) {
    if (int rc = require_sm100()) return rc;
    if (p.rows == 0 || p.hidden == 0) return BN_OK;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const bool add = p.b != nullptr;
    const int per_sm = p.hidden <= RN_THREADS * 8 ? 4 : 2;          // resident CTAs per SM; more rows loop
    const long long cap = (long long)sms * per_sm;
    const unsigned grid = (unsigned)(p.rows < cap ? p.rows : cap);
    cudaStream_t st = as_stream(stream);
    if (p.hidden <= RN_THREADS * 8) {
        if (add) rmsnorm_regs_kernel<8, true><<<grid, RN_THREADS, 0, st>>>(p);
        else rmsnorm_regs_kernel<8, false><<<grid, RN_THREADS, 0, st>>>(p);
    } else if (p.hidden <= RN_THREADS * RN_MAXV) {
        if (add) rmsnorm_regs_kernel<RN_MAXV, true><<<grid, RN_THREADS, 0, st>>>(p);
        else rmsnorm_regs_kernel<RN_MAXV, false><<<grid, RN_THREADS, 0, st>>>(p);
    } else {
        rmsnorm_wide_kernel<<<(unsigned)(p.rows < (long long)sms * 8 ? p.rows : (long long)sms * 8), RN_THREADS, 0, st>>>(p);
    }
    return launch_status(what);
}

}  // namespace bn

using namespace bn;

extern "C" int bn_rmsnorm_f32(const float* x, int64_t x_rs, int64_t x_cs, const float* w, int64_t w_cs, float* y,
                              int64_t y_rs, int64_t y_cs, int rows, int hidden, float eps, bn_stream_t stream) {
    if (!x || !w || !y) return fail(BN_ERR_INVALID_ARG, "bn_rmsnorm_f32: null pointer");
    if (rows < 0 || hidden < 0) return fail(BN_ERR_INVALID_ARG, "bn_rmsnorm_f32: bad shape rows=%d hidden=%d", rows, hidden);
    RmsParams p{x, x_rs, x_cs, nullptr, 0, 0, w, w_cs, nullptr, 0, 0, y, y_rs, y_cs, rows, hidden, eps};
    return rmsnorm_launch(p, stream, "bn_rmsnorm_f32");
}

extern "C" int bn_add_rmsnorm_f32(const float* a, int64_t a_rs, int64_t a_cs, const float* b, int64_t b_rs, int64_t b_cs,
                                  const float* w, int64_t w_cs, float* sum, int64_t s_rs, int64_t s_cs, float* y,
                                  int64_t y_rs, int64_t y_cs, int rows, int hidden, float eps, bn_stream_t stream) {
    if (!a || !b || !w || !y) return fail(BN_ERR_INVALID_ARG, "bn_add_rmsnorm_f32: null pointer");
    if (rows < 0 || hidden < 0)
        return fail(BN_ERR_INVALID_ARG, "bn_add_rmsnorm_f32: bad shape rows=%d hidden=%d", rows, hidden);
    RmsParams p{a, a_rs, a_cs, b, b_rs, b_cs, w, w_cs, sum, s_rs, s_cs, y, y_rs, y_cs, rows, hidden, eps};
    return rmsnorm_launch(p, stream, "bn_add_rmsnorm_f32");
}

// ---------------------------------------------------------------------------
// bf16 residual stream: s = a + b rounded to bf16 (the model dtype), y = s / sqrt(mean(s^2) + eps) * w with fp32
// arithmetic and one rounding of y.  Used by the bf16 decoder layer; no bit-compatibility constraint here, so the
// row is moved in 16-byte pieces and reduced with shuffles.
// ---------------------------------------------------------------------------
namespace bn {

struct RmsBf16Params {
    const __nv_bfloat16 *a, *b, *w;    // b may be null
    __nv_bfloat16 *s, *y;              // s may be null
    int rows, hidden;
    float eps;
};

constexpr int RB_MAXV = 2;             // 16-byte pieces per thread kept in registers: hidden <= 256 * 8 * 2 = 4096

__device__ __forceinline__ float bf16lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t packbf(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__global__ void __launch_bounds__(256)
rmsnorm_bf16_kernel(const RmsBf16Params p) {
    __shared__ float s_part[8];
    const int tid = threadIdx.x, lane = tid % 32, warp = tid / 32;
    const int pieces = p.hidden / 8;
    // Launched as a programmatic dependent: nothing is read before the kernel ahead of this one has completed.  The
    // kernel behind this one (a projection that first requests its weights into L2) may start now; it in turn waits
    // for this grid's completion before it reads anything written here.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const uint4* ar = reinterpret_cast<const uint4*>(p.a + (size_t)row * p.hidden);
        const uint4* br = p.b ? reinterpret_cast<const uint4*>(p.b + (size_t)row * p.hidden) : nullptr;
        uint4* sr = p.s ? reinterpret_cast<uint4*>(p.s + (size_t)row * p.hidden) : nullptr;
        uint4* yr = reinterpret_cast<uint4*>(p.y + (size_t)row * p.hidden);
        uint4 v[RB_MAXV];
        float acc = 0.f;
        auto fetch = [&](int c) {
            uint4 x = __ldg(ar + c);
            if (br) {
                const uint4 y4 = __ldg(br + c);
                uint32_t* xs = reinterpret_cast<uint32_t*>(&x);
                const uint32_t* ys = reinterpret_cast<const uint32_t*>(&y4);
#pragma unroll
                for (int e = 0; e < 4; ++e) xs[e] = packbf(bf16lo(xs[e]) + bf16lo(ys[e]), bf16hi(xs[e]) + bf16hi(ys[e]));
            }
            return x;
        };
        auto sq = [&](const uint4& x) {
            const uint32_t* xs = reinterpret_cast<const uint32_t*>(&x);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float lo = bf16lo(xs[e]), hi = bf16hi(xs[e]);
                acc = fmaf(lo, lo, acc);
                acc = fmaf(hi, hi, acc);
            }
        };
#pragma unroll
        for (int k = 0; k < RB_MAXV; ++k) {
            const int c = tid + k * 256;
            if (c < pieces) { v[k] = fetch(c); sq(v[k]); }
        }
        for (int c = tid + RB_MAXV * 256; c < pieces; c += 256) { const uint4 x = fetch(c); sq(x); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) s_part[warp] = acc;
        __syncthreads();
        float total = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < 8; ++w8) total += s_part[w8];
        const float inv = rsqrtf(total / (float)p.hidden + p.eps);
        auto emit = [&](int c, const uint4& x) {
            if (sr) sr[c] = x;
            const uint4 w4 = __ldg(reinterpret_cast<const uint4*>(p.w) + c);
            const uint32_t* xs = reinterpret_cast<const uint32_t*>(&x);
            const uint32_t* ws = reinterpret_cast<const uint32_t*>(&w4);
            uint4 o4;
            uint32_t* os = reinterpret_cast<uint32_t*>(&o4);
#pragma unroll
            for (int e = 0; e < 4; ++e)
                os[e] = packbf(bf16lo(xs[e]) * inv * bf16lo(ws[e]), bf16hi(xs[e]) * inv * bf16hi(ws[e]));
            yr[c] = o4;
        };
#pragma unroll
        for (int k = 0; k < RB_MAXV; ++k) {
            const int c = tid + k * 256;
            if (c < pieces) emit(c, v[k]);
        }
        for (int c = tid + RB_MAXV * 256; c < pieces; c += 256) emit(c, fetch(c));
        __syncthreads();     // s_part is rewritten by the next row
    }
}

}  // namespace bn

extern "C" int bn_add_rmsnorm_bf16(const void* a, const void* b, const void* w, void* sum, void* y, int rows, int hidden,
                                   float eps, bn_stream_t stream) {
    if (!a || !w || !y) return fail(BN_ERR_INVALID_ARG, "bn_add_rmsnorm_bf16: null pointer");
    if (rows < 0 || hidden < 0 || hidden % 8)
        return fail(BN_ERR_INVALID_ARG, "bn_add_rmsnorm_bf16: bad shape rows=%d hidden=%d (hidden must be a multiple of 8)",
                    rows, hidden);
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(w) |
         reinterpret_cast<uintptr_t>(sum) | reinterpret_cast<uintptr_t>(y)) & 15)
        return fail(BN_ERR_INVALID_ARG, "bn_add_rmsnorm_bf16: pointers must be 16-byte aligned");
    if (int rc = require_sm100()) return rc;
    if (rows == 0 || hidden == 0) return BN_OK;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long cap = (long long)sms * 8;
    RmsBf16Params p{static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b),
                    static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(sum),
                    static_cast<__nv_bfloat16*>(y), rows, hidden, eps};
    launch_dependent(rmsnorm_bf16_kernel, (unsigned)(rows < cap ? rows : cap), 256, 0, as_stream(stream), p);
    return launch_status("bn_add_rmsnorm_bf16");
}

// Device-side token embedding gather and per-row argmax, so that generate() neither uploads a gathered embedding
// matrix nor downloads the logits.
//
//   bn_embedding_gather_f32  out[i, :] = table[ids[i], :]
//       reference: LLaMAModel.embed gathers on the HOST, row by row, from a device-to-host copy of the whole table
//       (262 MB for TinyLLaMA) and uploads the result (mygrad/llama/llama_model.py:58-78)
//   bn_argmax_rows_f32       out[r] = index of the first maximum of row r
//       reference: op_argmax (src/ops/op_reduction.cuh:196-210) with MaxAccumFunc (:5-19): accum = x[0]; a later
//       element replaces it only if it is strictly greater, so ties keep the first index and a NaN never wins unless
//       it is element 0.  The reference runs ONE THREAD per row; here a CTA per row.
// Both are HBM-bound copies / reductions: 16-byte accesses, consecutive threads on consecutive addresses.
#include "common.cuh"

namespace bn {

__global__ void __launch_bounds__(256)
embedding_gather_kernel(const float* __restrict__ table, int64_t table_rs, const uint32_t* __restrict__ ids,
                        float* __restrict__ out, int64_t out_rs, int n_ids, int hidden, int vocab,
                        int* __restrict__ error_word) {
    for (int i = blockIdx.x; i < n_ids; i += gridDim.x) {
        const uint32_t id = ids[i];
        const bool valid = id < (uint32_t)vocab;
        if (!valid && threadIdx.x == 0 && error_word) atomicExch(error_word, BN_ERR_INVALID_ARG);
        const float* src = table + (int64_t)(valid ? id : 0) * table_rs;
        float* dst = out + (int64_t)i * out_rs;
        const bool vec = (hidden % 4 == 0) && (table_rs % 4 == 0) && (out_rs % 4 == 0) &&
                         ((reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
        if (vec) {
            const float4* s4 = reinterpret_cast<const float4*>(src);
            float4* d4 = reinterpret_cast<float4*>(dst);
            for (int c = threadIdx.x; c < hidden / 4; c += blockDim.x)
                d4[c] = valid ? __ldg(s4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = valid ? __ldg(src + c) : 0.f;
        }
    }
}

// (value, index) with the reference's order: strictly greater wins, ties keep the smaller index, NaN never wins
struct ArgMax {
    float v;
    int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__global__ void __launch_bounds__(256)
argmax_rows_kernel(const float* __restrict__ x, int64_t x_rs, int64_t x_cs, uint32_t* __restrict__ out, int rows,
                   int cols) {
    __shared__ float sv[8];
    __shared__ int si[8];
    const int tid = threadIdx.x, lane = tid % 32, warp = tid / 32;
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* xr = x + (int64_t)r * x_rs;
        ArgMax best{-INFINITY, 0x7fffffff};
        if (x_cs == 1 && (reinterpret_cast<uintptr_t>(xr) & 15) == 0) {
            const float4* x4 = reinterpret_cast<const float4*>(xr);
            for (int c = tid; c < cols / 4; c += blockDim.x) {
                const float4 v = __ldg(x4 + c);
                best = better(best, ArgMax{v.x, 4 * c});
                best = better(best, ArgMax{v.y, 4 * c + 1});
                best = better(best, ArgMax{v.z, 4 * c + 2});
                best = better(best, ArgMax{v.w, 4 * c + 3});
            }
            for (int c = cols / 4 * 4 + tid; c < cols; c += blockDim.x) best = better(best, ArgMax{__ldg(xr + c), c});
        } else {
            for (int c = tid; c < cols; c += blockDim.x) best = better(best, ArgMax{__ldg(xr + (int64_t)c * x_cs), c});
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax other{__shfl_down_sync(0xffffffffu, best.v, o), __shfl_down_sync(0xffffffffu, best.i, o)};
            best = better(best, other);
        }
        if (lane == 0) { sv[warp] = best.v; si[warp] = best.i; }
        __syncthreads();
        if (tid == 0) {
            ArgMax b{sv[0], si[0]};
            for (int w = 1; w < 8; ++w) b = better(b, ArgMax{sv[w], si[w]});
            // the reference starts from element 0: it stays unless something is strictly greater; a NaN there
            // is never beaten, and if no element compares (all NaN or -inf) index 0 stands
            const float x0 = __ldg(xr);
            out[r] = (x0 != x0 || !(b.v > x0)) ? 0u : (uint32_t)b.i;
        }
        __syncthreads();
    }
}

}  // namespace bn

using namespace bn;

extern "C" int bn_embedding_gather_f32(const float* table, int64_t table_rs, const uint32_t* ids, float* out,
                                       int64_t out_rs, int n_ids, int hidden, int vocab, int* error_word,
                                       bn_stream_t stream) {
    if (!table || !ids || !out) return fail(BN_ERR_INVALID_ARG, "bn_embedding_gather_f32: null pointer");
    if (n_ids < 0 || hidden < 0 || vocab <= 0)
        return fail(BN_ERR_INVALID_ARG, "bn_embedding_gather_f32: bad shape n_ids=%d hidden=%d vocab=%d", n_ids, hidden, vocab);
    if (int rc = require_sm100()) return rc;
    if (n_ids == 0 || hidden == 0) return BN_OK;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long cap = (long long)sms * 8;
    embedding_gather_kernel<<<(unsigned)(n_ids < cap ? n_ids : cap), 256, 0, as_stream(stream)>>>(
        table, table_rs, ids, out, out_rs, n_ids, hidden, vocab, error_word);
    return launch_status("bn_embedding_gather_f32");
}

extern "C" int bn_argmax_rows_f32(const float* x, int64_t x_rs, int64_t x_cs, uint32_t* out, int rows, int cols,
                                  bn_stream_t stream) {
    if (!x || !out) return fail(BN_ERR_INVALID_ARG, "bn_argmax_rows_f32: null pointer");
    if (rows < 0 || cols <= 0) return fail(BN_ERR_INVALID_ARG, "bn_argmax_rows_f32: bad shape rows=%d cols=%d", rows, cols);
    if (int rc = require_sm100()) return rc;
    if (rows == 0) return BN_OK;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long cap = (long long)sms * 8;
    argmax_rows_kernel<<<(unsigned)(rows < cap ? rows : cap), 256, 0, as_stream(stream)>>>(x, x_rs, x_cs, out, rows, cols);
    return launch_status("bn_argmax_rows_f32");
}

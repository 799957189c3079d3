// Paged bf16 KV cache: the append step.
//
// The reference keeps no cache (mygrad/llama/llama_model.py:136-144 recomputes
// the whole sequence per generated token); this is the new layout that makes
// single-token decode possible.  One pool per layer:
//     pool[page][kv_head][0 = K, 1 = V][16 tokens][64]   bf16
// so that K and V of one (page, head) are one contiguous 4 KB block that the
// decode kernel fetches with a single TMA box.  K is stored already rotated
// (src/ops/op_rope.cuh:55-99 at the token's position), V as is.
#include "common.cuh"
#include "ptx.cuh"

namespace bn {

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// one thread per (token, kv head, pair)
template <typename T>
__global__ void kv_append_kernel(__nv_bfloat16* __restrict__ pool, int64_t pool_pages,
                                 const int32_t* __restrict__ page_table, int max_pages,
                                 const int32_t* __restrict__ seq_ids, const int32_t* __restrict__ positions, int T_,
                                 const T* __restrict__ k_new, const T* __restrict__ v_new, int64_t row_stride, int Hkv,
                                 int D, float theta) {
    const int half = D / 2;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    // launched as a programmatic dependent: the projections that produce k_new / v_new have completed after the wait;
    // the decode kernel behind this one may begin its set-up and waits for this grid before it reads the pool
    ptx::grid_dependency_wait();
    ptx::grid_launch_dependents();
    if (idx >= (int64_t)T_ * Hkv * half) return;
    const int i = (int)(idx % half);
    const int g = (int)((idx / half) % Hkv);
    const int t = (int)(idx / ((int64_t)half * Hkv));
    const int pos = positions[t];
    const int lp = pos / BN_PAGE_TOKENS;
    if (pos < 0 || lp >= max_pages) return;
    const int page = page_table[(int64_t)seq_ids[t] * max_pages + lp];
    if (page < 0 || page >= pool_pages) return;
    const int slot = pos % BN_PAGE_TOKENS;
    const T* kp = k_new + t * row_stride + g * D + 2 * i;
    const T* vp = v_new + t * row_stride + g * D + 2 * i;
    const float x0 = load_as_float(kp), x1 = load_as_float(kp + 1);
    const float freq = rope_inv_freq(i, D, theta);
    const float angle = pos * freq;
    const float cos_angle = cosf(angle), sin_angle = sinf(angle);
    const float y0 = x0 * cos_angle - x1 * sin_angle;
    const float y1 = x0 * sin_angle + x1 * cos_angle;
    __nv_bfloat16* kdst = pool + ((((int64_t)page * Hkv + g) * 2 + 0) * BN_PAGE_TOKENS + slot) * D + 2 * i;
    __nv_bfloat16* vdst = pool + ((((int64_t)page * Hkv + g) * 2 + 1) * BN_PAGE_TOKENS + slot) * D + 2 * i;
    *reinterpret_cast<uint32_t*>(kdst) = ptx::pack_bf16(y0, y1);
    *reinterpret_cast<uint32_t*>(vdst) = ptx::pack_bf16(load_as_float(vp), load_as_float(vp + 1));
}

}  // namespace bn

using namespace bn;

extern "C" int bn_kv_append(void* pool, int64_t pool_pages, const int32_t* page_table, int max_pages,
                            const int32_t* seq_ids, const int32_t* positions, int T, const void* k_new,
                            const void* v_new, int64_t kv_row_stride, int dtype, int Hkv, int D, float theta,
                            bn_stream_t stream) {
    if (!pool || !page_table || !seq_ids || !positions || !k_new || !v_new)
        return fail(BN_ERR_INVALID_ARG, "bn_kv_append: null pointer");
    if (T < 0 || Hkv <= 0 || D <= 0 || D % 2 || max_pages <= 0 || pool_pages <= 0)
        return fail(BN_ERR_INVALID_ARG, "bn_kv_append: bad sizes T=%d Hkv=%d D=%d max_pages=%d", T, Hkv, D, max_pages);
    if (dtype != 0 && dtype != 1) return fail(BN_ERR_INVALID_ARG, "bn_kv_append: dtype=%d (0 = fp32, 1 = bf16)", dtype);
    if (int rc = require_sm100()) return rc;
    if (T == 0) return BN_OK;
    const int64_t n = (int64_t)T * Hkv * (D / 2);
    const unsigned blocks = (unsigned)((n + 255) / 256);
    __nv_bfloat16* pl = static_cast<__nv_bfloat16*>(pool);
    if (dtype == 0)
        launch_dependent(kv_append_kernel<float>, blocks, 256, 0, as_stream(stream), pl, pool_pages, page_table,
                         max_pages, seq_ids, positions, T, static_cast<const float*>(k_new),
                         static_cast<const float*>(v_new), kv_row_stride, Hkv, D, theta);
    else
        launch_dependent(kv_append_kernel<__nv_bfloat16>, blocks, 256, 0, as_stream(stream), pl, pool_pages, page_table,
                         max_pages, seq_ids, positions, T, static_cast<const __nv_bfloat16*>(k_new),
                         static_cast<const __nv_bfloat16*>(v_new), kv_row_stride, Hkv, D, theta);
    return launch_status("bn_kv_append");
}

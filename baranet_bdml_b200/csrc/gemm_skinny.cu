// C (M,N) bf16 = A (M,K) bf16 @ Bt (N,K)^T bf16 for M <= 16 rows: the projections of a decode step, where every
// sequence contributes ONE row (mygrad/llama/llama_layers.py:157-159,186 and the MLP, :217-232, applied to the new
// token only; reference operator op_mm, src/ops/op_mm.cuh:39-57, whose naive kernel runs for such shapes).
//
// With so few rows the product is a stream of the weight matrix through the SMs: 2 FLOP per weight byte and row, far
// below what the tensor cores need, so the bound is HBM bandwidth and what matters is that every SM has many loads in
// flight.  The 128-row tcgen05 tiles of the large GEMM are the wrong tool here (an eighth of each instruction would do
// useful work and a tile's ring holds few bytes in flight); this kernel uses warp-level mma.sync.m16n8k16, whose M = 16
// is the whole batch:
//   CTA = 8 warps = 8 output columns (8 rows of Bt); warp w takes the w-th eighth of K for all 8 columns.
//   A lane loads 16 contiguous bytes (8 bf16 along K) of ONE weight row and of two activation rows per 32-wide K step
//   (in batches of 4 or 8 steps, weight and activation loads of a batch all in flight before the first use).  The K order inside a step
//   is whatever this lane assignment gives: a dot product does not care, as long as A and B use the same one, so no
//   shuffles or shared-memory staging are needed to form the MMA fragments.
//   The 8 warps' partial sums (16 x 8 fp32) are added through shared memory in warp order (deterministic).
// Variants: up to three column ranges of one concatenated weight written to separate outputs (q, k, v of the layer in one
// launch); the same with the K and V ranges rotated / appended to the paged cache by the epilogue instead (what
// bn_kv_append would do with them, mygrad/llama/llama_layers.py:161-171 for the new token); and the SwiGLU pair (two weights, h = silu(x Wg) * (x Wu), op_silu.cuh:7-15).
// K must be a multiple of 256 (a warp's eighth is a whole number of 32-wide steps) and at most 8192; N a multiple
// of 8.  Anything else belongs to bn_gemm_bf16_nt_small_m.
#include "common.cuh"
#include "ptx.cuh"

namespace bn {

using namespace ptx;

constexpr int SK_WARPS = 8;
constexpr int SK_MAX_STEPS = 32;        // 32-wide K steps per warp: K <= 8 * 32 * 32 = 8192

struct SkinnyParams {
    const __nv_bfloat16* a;             // (M, K)
    const __nv_bfloat16* bt;            // (N, K)
    const __nv_bfloat16* bt2;           // SwiGLU: the up weight (N, K); bt is the gate weight
    __nv_bfloat16* out[3];              // outputs of the column ranges
    int n_end[3];                       // range r covers columns [n_end[r-1], n_end[r])
    int ld[3];                          // row stride of out[r] in elements
    int M, N, K, steps;                 // steps = K / (8 * 32)
    // APPEND: columns from n_end[0] on are the K and V projections of one new token per row and go to the paged cache
    // instead of out[1] / out[2] (arguments as bn_kv_append)
    __nv_bfloat16* pool;
    const int32_t* page_table;
    const int32_t* seq_ids;
    const int32_t* positions;
    int64_t pool_pages;
    int max_pages, Hkv, D;
    float theta;
};

// CH = K steps whose loads a lane keeps in flight at once.  More of them cover more latency per warp; fewer leave
// registers for more CTAs per SM (8: two, 2: four), which matters when the grid would otherwise need a second, nearly
// empty wave.
template <bool SWIGLU, int CH, bool APPEND = false>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(const SkinnyParams p) {
    __shared__ float s_part[SK_WARPS][2][16][8 + 1];
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int g = lane / 4, j = lane % 4;                 // weight row inside the CTA's 8 / which 8 of a step's 32 K positions
    const int n0 = blockIdx.x * 8;
    const size_t kbase = (size_t)warp * p.steps * 32 + j * 8;
    const uint4* bw = reinterpret_cast<const uint4*>(p.bt + (size_t)(n0 + g) * p.K + kbase);
    const uint4* bw2 = SWIGLU ? reinterpret_cast<const uint4*>(p.bt2 + (size_t)(n0 + g) * p.K + kbase) : nullptr;
    const uint4* a_lo = reinterpret_cast<const uint4*>(p.a + (size_t)g * p.K + kbase);
    const uint4* a_hi = reinterpret_cast<const uint4*>(p.a + (size_t)(g + 8) * p.K + kbase);
    const bool lo_ok = g < p.M, hi_ok = g + 8 < p.M;
    float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
    // Loads first, arithmetic after: for a batch of K steps the lane requests its pieces of the weight rows (evict-first:
    // each weight byte is read once per launch) AND of the two activation rows (read by every CTA, so they stay in L2)
    // before it uses any of them - a launch of this kernel is one or two memory round trips long, and a load issued after
    // a wait would add its whole latency to that.
    const uint4 z = make_uint4(0, 0, 0, 0);
    uint4 wv[CH], wv2[SWIGLU ? CH : 1], al[CH], ah[CH];
    auto load_weights = [&](int s0) {
#pragma unroll
        for (int s = 0; s < CH; ++s)
            if (s0 + s < p.steps) {
                wv[s] = __ldcs(bw + (size_t)(s0 + s) * 4);              // 32 K positions = 64 B = 4 x 16 B per row and step
                if (SWIGLU) wv2[s] = __ldcs(bw2 + (size_t)(s0 + s) * 4);
            }
    };
    // The warp's whole slice of the 8 weight rows is requested into L2 at once (a 128-byte line is two steps of a
    // row; the four lanes of a row name the same line and are merged): the batches below then find their weights
    // in L2 instead of each paying a round trip to HBM.  Under a programmatic dependent launch this happens while the
    // kernel before this one in the stream is still running - the weights do not depend on it, the activations do,
    // and nothing is READ before the wait (L2 is the point of coherence, so a line prefetched early cannot go stale).
    for (int s = 0; s < p.steps; s += 2) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(bw + (size_t)s * 4));
        if (SWIGLU) asm volatile("prefetch.global.L2 [%0];" ::"l"(bw2 + (size_t)s * 4));
    }
    grid_dependency_wait();
    grid_launch_dependents();
    for (int s0 = 0; s0 < p.steps; s0 += CH) {
        load_weights(s0);
#pragma unroll
        for (int s = 0; s < CH; ++s)
            if (s0 + s < p.steps) {
                al[s] = lo_ok ? __ldg(a_lo + (size_t)(s0 + s) * 4) : z;
                ah[s] = hi_ok ? __ldg(a_hi + (size_t)(s0 + s) * 4) : z;
            }
#pragma unroll
        for (int s = 0; s < CH; ++s)
            if (s0 + s < p.steps) {
                // two k16 MMAs per step: the lane's first four K positions play (2j, 2j+1, 2j+8, 2j+9) of the first,
                // its last four of the second, in A and B alike
                mma_bf16_16816(acc, al[s].x, ah[s].x, al[s].y, ah[s].y, wv[s].x, wv[s].y);
                mma_bf16_16816(acc, al[s].z, ah[s].z, al[s].w, ah[s].w, wv[s].z, wv[s].w);
                if (SWIGLU) {
                    mma_bf16_16816(acc2, al[s].x, ah[s].x, al[s].y, ah[s].y, wv2[s].x, wv2[s].y);
                    mma_bf16_16816(acc2, al[s].z, ah[s].z, al[s].w, ah[s].w, wv2[s].z, wv2[s].w);
                }
            }
    }
    // C fragment: acc[0], acc[1] = row g, columns 2j, 2j+1; acc[2], acc[3] = row g + 8
    s_part[warp][0][g][2 * j] = acc[0];
    s_part[warp][0][g][2 * j + 1] = acc[1];
    s_part[warp][0][g + 8][2 * j] = acc[2];
    s_part[warp][0][g + 8][2 * j + 1] = acc[3];
    if (SWIGLU) {
        s_part[warp][1][g][2 * j] = acc2[0];
        s_part[warp][1][g][2 * j + 1] = acc2[1];
        s_part[warp][1][g + 8][2 * j] = acc2[2];
        s_part[warp][1][g + 8][2 * j + 1] = acc2[3];
    }
    __syncthreads();
    if (threadIdx.x < 128) {
        const int row = threadIdx.x / 8, col = threadIdx.x % 8;
        float v = 0.f, u = 0.f;
        if (row < p.M) {
#pragma unroll
            for (int w = 0; w < SK_WARPS; ++w) {
                v += s_part[w][0][row][col];
                if (SWIGLU) u += s_part[w][1][row][col];
            }
            if (SWIGLU) v = __fdividef(v, 1.f + __expf(-v)) * u;          // silu(gate) * up
        }
        const int n = n0 + col;
        if (APPEND && n >= p.n_end[0]) {       // the same for the CTA's 8 columns: the ranges are multiples of 8
            // What bn_kv_append does with the bf16 row the plain kernel would have written: the value is rounded to
            // bf16 first, a K pair (2i, 2i+1) = (this column, its neighbour) is rotated at the row's position in fp32
            // and rounded again, V is stored as it is - the cache ends up with the bits of the two-launch path.
            const float vb = __bfloat162float(__float2bfloat16(v));
            const float other = __shfl_xor_sync(0xffffffffu, vb, 1);
            if (row < p.M) {
                const bool is_k = n < p.n_end[1];
                const int local = n - (is_k ? p.n_end[0] : p.n_end[1]);
                const int g = local / p.D, d = local - g * p.D;
                const int pos = p.positions[row];
                const int lp = pos / BN_PAGE_TOKENS;
                if (pos >= 0 && lp < p.max_pages) {
                    const int page = p.page_table[(int64_t)p.seq_ids[row] * p.max_pages + lp];
                    if (page >= 0 && page < p.pool_pages) {
                        float y = vb;
                        if (is_k) {
                            const float angle = pos * rope_inv_freq(d / 2, p.D, p.theta);
                            const float c = cosf(angle), sn = sinf(angle);
                            y = (d & 1) ? other * sn + vb * c : vb * c - other * sn;
                        }
                        p.pool[((((int64_t)page * p.Hkv + g) * 2 + (is_k ? 0 : 1)) * BN_PAGE_TOKENS + pos % BN_PAGE_TOKENS) * p.D + d] =
                            __float2bfloat16(y);
                    }
                }
            }
        } else if (row < p.M) {
            // selects, not indexed parameter arrays (an index known only at run time would copy them to local memory)
            __nv_bfloat16* o = p.out[0];
            int ld = p.ld[0], first = 0;
            if (n >= p.n_end[1]) { o = p.out[2]; ld = p.ld[2]; first = p.n_end[1]; }
            else if (n >= p.n_end[0]) { o = p.out[1]; ld = p.ld[1]; first = p.n_end[0]; }
            o[(size_t)row * ld + (n - first)] = __float2bfloat16(v);
        }
    }
}

static int skinny_check(const char* what, const void* a, const void* bt, int M, int N, int K) {
    if (!a || !bt) return fail(BN_ERR_INVALID_ARG, "%s: null pointer", what);
    if (M <= 0 || M > 16) return fail(BN_ERR_UNSUPPORTED, "%s: M=%d (1..16 rows)", what, M);
    if (N <= 0 || N % 8) return fail(BN_ERR_UNSUPPORTED, "%s: N=%d must be a positive multiple of 8", what, N);
    if (K <= 0 || K % 256 || K > SK_WARPS * 32 * SK_MAX_STEPS)
        return fail(BN_ERR_UNSUPPORTED, "%s: K=%d must be a multiple of 256, at most %d", what, K, SK_WARPS * 32 * SK_MAX_STEPS);
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(bt)) & 15)
        return fail(BN_ERR_INVALID_ARG, "%s: a/bt must be 16-byte aligned", what);
    return require_sm100();
}

}  // namespace bn

using namespace bn;

extern "C" int bn_gemm_bf16_nt_skinny(const void* a, const void* bt, int M, int N, int K, void* out0, int n0, void* out1,
                                      int n1, void* out2, bn_stream_t stream) {
    const char* what = "bn_gemm_bf16_nt_skinny";
    if (int rc = skinny_check(what, a, bt, M, N, K)) return rc;
    if (!out0 || n0 <= 0 || n0 > N || n0 % 8 || n1 < 0 || n1 % 8 || n0 + n1 > N || (n1 > 0 && !out1) ||
        (n0 + n1 < N && !out2))
        return fail(BN_ERR_INVALID_ARG, "%s: column ranges %d + %d of %d need their outputs (multiples of 8)", what, n0, n1, N);
    SkinnyParams p{};
    p.a = static_cast<const __nv_bfloat16*>(a);
    p.bt = static_cast<const __nv_bfloat16*>(bt);
    p.bt2 = nullptr;
    p.out[0] = static_cast<__nv_bfloat16*>(out0);
    p.out[1] = static_cast<__nv_bfloat16*>(out1);
    p.out[2] = static_cast<__nv_bfloat16*>(out2);
    p.n_end[0] = n0; p.n_end[1] = n0 + n1; p.n_end[2] = N;
    p.ld[0] = n0; p.ld[1] = n1; p.ld[2] = N - n0 - n1;
    p.M = M; p.N = N; p.K = K; p.steps = K / (SK_WARPS * 32);
    // measured on the decode step's shapes: 256 CTAs (o, down) run fastest two per SM with 8 steps in flight, 320 (q/k/v
    // in one launch) four per SM with 2
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (N / 8 <= 2 * sms) launch_dependent(gemm_skinny_kernel<false, 8>, N / 8, SK_WARPS * 32, 0, as_stream(stream), p);
    else launch_dependent(gemm_skinny_kernel<false, 2>, N / 8, SK_WARPS * 32, 0, as_stream(stream), p);
    return launch_status(what);
}

extern "C" int bn_gemm_swiglu_bf16_nt_skinny(const void* x, const void* gate_t, const void* up_t, void* h, int M, int inter,
                                             int K, bn_stream_t stream) {
    const char* what = "bn_gemm_swiglu_bf16_nt_skinny";
    if (int rc = skinny_check(what, x, gate_t, M, inter, K)) return rc;
    if (!up_t || !h || (reinterpret_cast<uintptr_t>(up_t) & 15)) return fail(BN_ERR_INVALID_ARG, "%s: null or misaligned pointer", what);
    SkinnyParams p{};
    p.a = static_cast<const __nv_bfloat16*>(x);
    p.bt = static_cast<const __nv_bfloat16*>(gate_t);
    p.bt2 = static_cast<const __nv_bfloat16*>(up_t);
    p.out[0] = static_cast<__nv_bfloat16*>(h);
    p.out[1] = p.out[2] = nullptr;
    p.n_end[0] = p.n_end[1] = p.n_end[2] = inter;
    p.ld[0] = inter; p.ld[1] = p.ld[2] = 0;
    p.M = M; p.N = inter; p.K = K; p.steps = K / (SK_WARPS * 32);
    launch_dependent(gemm_skinny_kernel<true, 2>, inter / 8, SK_WARPS * 32, 0, as_stream(stream), p);
    return launch_status(what);
}

extern "C" int bn_gemm_qkv_append_bf16_skinny(const void* x, const void* wqkv_t, int M, int hidden, int Hq, int Hkv, int D,
                                              void* q_out, void* pool, int64_t pool_pages, const int32_t* page_table,
                                              int max_pages, const int32_t* seq_ids, const int32_t* positions, float theta,
                                              bn_stream_t stream) {
    const char* what = "bn_gemm_qkv_append_bf16_skinny";
    if (Hq <= 0 || Hkv <= 0 || D <= 0 || D % 8)
        return fail(BN_ERR_INVALID_ARG, "%s: bad head shape Hq=%d Hkv=%d D=%d (D a multiple of 8)", what, Hq, Hkv, D);
    const int N = (Hq + 2 * Hkv) * D;
    if (int rc = skinny_check(what, x, wqkv_t, M, N, hidden)) return rc;
    if (!q_out || !pool || !page_table || !seq_ids || !positions || max_pages <= 0 || pool_pages <= 0)
        return fail(BN_ERR_INVALID_ARG, "%s: null pointer or empty cache", what);
    SkinnyParams p{};
    p.a = static_cast<const __nv_bfloat16*>(x);
    p.bt = static_cast<const __nv_bfloat16*>(wqkv_t);
    p.out[0] = static_cast<__nv_bfloat16*>(q_out);
    p.n_end[0] = Hq * D; p.n_end[1] = (Hq + Hkv) * D; p.n_end[2] = N;
    p.ld[0] = Hq * D;
    p.M = M; p.N = N; p.K = hidden; p.steps = hidden / (SK_WARPS * 32);
    p.pool = static_cast<__nv_bfloat16*>(pool);
    p.page_table = page_table; p.seq_ids = seq_ids; p.positions = positions;
    p.pool_pages = pool_pages; p.max_pages = max_pages; p.Hkv = Hkv; p.D = D; p.theta = theta;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (N / 8 <= 2 * sms) launch_dependent(gemm_skinny_kernel<false, 8, true>, N / 8, SK_WARPS * 32, 0, as_stream(stream), p);
    else launch_dependent(gemm_skinny_kernel<false, 2, true>, N / 8, SK_WARPS * 32, 0, as_stream(stream), p);
    return launch_status(what);
}

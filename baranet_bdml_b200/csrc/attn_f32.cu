// fp32 path: operators whose arithmetic ORDER matches the reference's fp32 SIMT
// kernels, so that results agree with it far inside the 1e-5 gate instead of
// merely within rounding noise of the exact answer.
//
//   bn_mm_f32            one FMA chain per output, k ascending
//                        (reference: src/ops/op_mm_optimized.cuh:35-62)
//   bn_rope_f32          reference: src/ops/op_rope.cuh:55-99
//   bn_attn_prefill_f32  rope -> q k^T -> *scale -> causal softmax -> p v fused
//                        in one launch, no (S,S) matrix in memory
//                        (reference sequence: mygrad/llama/llama_layers.py:161-183)
//
// These are parity kernels (small S, fp32); the roofline targets are the bf16
// kernels in attn_prefill_sm100.cu and attn_decode.cu.
#include "common.cuh"

namespace bn {

// ---------------------------------------------------------------------------
// GEMM: 64x64 output tile, 256 threads, 4x4 outputs per thread, k in slabs of 16
// ---------------------------------------------------------------------------
constexpr int MM_T = 64;
constexpr int MM_K = 16;

__global__ void __launch_bounds__(256)
mm_f32_kernel(const float* __restrict__ A, int64_t a_rs, int64_t a_cs, const float* __restrict__ B, int64_t b_rs,
              int64_t b_cs, float* __restrict__ C, int64_t c_rs, int64_t c_cs, int M, int K, int N) {
    __shared__ float As[MM_K][MM_T + 4];
    __shared__ float Bs[MM_K][MM_T + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int row0 = blockIdx.y * MM_T, col0 = blockIdx.x * MM_T;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += MM_K) {
        // stage A (64 rows x 16 k) and B (16 k x 64 cols); out-of-range -> 0
#pragma unroll
        for (int e = tid; e < MM_T * MM_K; e += 256) {
            int kk = e % MM_K, r = e / MM_K;
            int gr = row0 + r, gk = k0 + kk;
            As[kk][r] = (gr < M && gk < K) ? A[gr * a_rs + gk * a_cs] : 0.0f;
        }
#pragma unroll
        for (int e = tid; e < MM_T * MM_K; e += 256) {
            int c = e % MM_T, kk = e / MM_T;
            int gc = col0 + c, gk = k0 + kk;
            Bs[kk][c] = (gc < N && gk < K) ? B[gk * b_rs + gc * b_cs] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MM_K; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int gr = row0 + ty * 4 + i;
        if (gr >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int gc = col0 + tx * 4 + j;
            if (gc < N) C[gr * c_rs + gc * c_cs] = acc[i][j];
        }
    }
}

// ---------------------------------------------------------------------------
// RoPE, one thread per adjacent pair
// ---------------------------------------------------------------------------
__global__ void rope_f32_kernel(const float* __restrict__ x, int64_t x_rs, int64_t x_cs, float* __restrict__ y,
                                int64_t y_rs, int64_t y_cs, int rows, int cols, int head_dim, float theta,
                                int position_offset) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int pairs_per_row = cols / 2;
    if (idx >= (int64_t)rows * pairs_per_row) return;
    int row = (int)(idx / pairs_per_row);
    int c0 = (int)(idx % pairs_per_row) * 2;
    int pair = (c0 % head_dim) / 2;
    int position = row + position_offset;
    float freq = rope_inv_freq(pair, head_dim, theta);
    float angle = position * freq;
    float cos_angle = cosf(angle), sin_angle = sinf(angle);
    float x0 = x[row * x_rs + c0 * x_cs], x1 = x[row * x_rs + (c0 + 1) * x_cs];
    y[row * y_rs + c0 * y_cs] = x0 * cos_angle - x1 * sin_angle;
    y[row * y_rs + (c0 + 1) * y_cs] = x0 * sin_angle + x1 * cos_angle;
}

// ---------------------------------------------------------------------------
// Fused attention core, fp32, two passes over the keys
// ---------------------------------------------------------------------------
constexpr int AF_BM = 16;    // query rows per CTA
constexpr int AF_BN = 64;    // keys per tile
constexpr int AF_BK = 32;    // dot-product columns staged per step
constexpr int AF_MAXHALF = 32;   // head_dim <= 64
constexpr int AF_MAXOUT = 16;    // distinct output columns per problem <= 256

struct AttnF32Params {
    const float *q, *k, *v;
    float* out;
    int64_t q_rs, q_cs, k_rs, k_cs, v_rs, v_cs, o_rs, o_cs;
    int S, Hq, Hkv, D;
    float scale, theta;
    int position_offset, causal, heads_mode, apply_rope;
};

// Column c of the (virtual) repeated K/V matrix -> column of the stored one.
__device__ __forceinline__ int kv_col(int c, int D, int n_rep) { return (c / D / n_rep) * D + c % D; }

__global__ void __launch_bounds__(256) attn_f32_kernel(AttnF32Params p) {
    __shared__ float Qs[AF_BM][AF_BK];
    __shared__ float Ks[AF_BN][AF_BK + 1];
    __shared__ float Ps[AF_BM][AF_BN];
    __shared__ float cq[AF_BM][AF_MAXHALF], sq[AF_BM][AF_MAXHALF];
    __shared__ float ck[AF_BN][AF_MAXHALF], sk[AF_BN][AF_MAXHALF];
    __shared__ float inv_freq[AF_MAXHALF];

    const int tid = threadIdx.x;
    const int r = tid / 16, cg = tid % 16;
    const int row0 = blockIdx.x * AF_BM;
    const int D = p.D, half = D / 2, n_rep = p.Hq / p.Hkv;
    // problem = the set of columns one softmax spans
    const int prob = blockIdx.y;
    const bool collapsed = p.heads_mode == BN_HEADS_COLLAPSED;
    const int qc0 = collapsed ? 0 : prob * D;              // first q column of the dot product
    const int Wd = collapsed ? p.Hq * D : D;               // dot-product width
    const int vc0 = collapsed ? 0 : (prob / n_rep) * D;    // first stored V column of the output
    const int Wo = collapsed ? p.Hkv * D : D;              // distinct output columns

    if (tid < half) inv_freq[tid] = rope_inv_freq(tid, D, p.theta);
    __syncthreads();
    if (p.apply_rope) {
        for (int e = tid; e < AF_BM * half; e += 256) {
            int rr = e / half, i = e % half;
            float angle = (row0 + rr + p.position_offset) * inv_freq[i];
            cq[rr][i] = cosf(angle);
            sq[rr][i] = sinf(angle);
        }
    }
    const int grow = row0 + r;
    // last valid key for this CTA's rows / for this thread's row
    int block_last = p.causal ? min(p.S - 1, row0 + AF_BM - 1 + p.position_offset) : p.S - 1;
    int row_last = p.causal ? min(p.S - 1, grow + p.position_offset) : p.S - 1;
    if (grow >= p.S) row_last = -1;
    const int n_tiles = block_last >= 0 ? block_last / AF_BN + 1 : 0;

    float m_run = -INFINITY, l_run = 0.0f;
    float acc[AF_MAXOUT];
#pragma unroll
    for (int j = 0; j < AF_MAXOUT; ++j) acc[j] = 0.0f;

    for (int pass = 0; pass < 2; ++pass) {
        for (int jt = 0; jt < n_tiles; ++jt) {
            const int j0 = jt * AF_BN;
            __syncthreads();  // previous tile's Ps / ck readers are done
            if (p.apply_rope) {
                for (int e = tid; e < AF_BN * half; e += 256) {
                    int jj = e / half, i = e % half;
                    float angle = (j0 + jj + p.position_offset) * inv_freq[i];
                    ck[jj][i] = cosf(angle);
                    sk[jj][i] = sinf(angle);
                }
            }
            float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int c0 = 0; c0 < Wd; c0 += AF_BK) {
                __syncthreads();
                // stage rotated Q (16 x 32) and rotated K (64 x 32), pair-wise
                for (int e = tid; e < (AF_BM + AF_BN) * (AF_BK / 2); e += 256) {
                    int pr = e % (AF_BK / 2), rr = e / (AF_BK / 2);
                    int c = c0 + 2 * pr;             // even column inside the dot product
                    bool isq = rr < AF_BM;
                    int lr = isq ? rr : rr - AF_BM;
                    int g = isq ? row0 + lr : j0 + lr;
                    float x0 = 0.0f, x1 = 0.0f;
                    if (g < p.S && c < Wd) {
                        if (isq) {
                            x0 = p.q[g * p.q_rs + (qc0 + c) * p.q_cs];
                            x1 = p.q[g * p.q_rs + (qc0 + c + 1) * p.q_cs];
                        } else {
                            int kc = kv_col(qc0 + c, D, n_rep);
                            x0 = p.k[g * p.k_rs + kc * p.k_cs];
                            x1 = p.k[g * p.k_rs + (kc + 1) * p.k_cs];
                        }
                    }
                    float y0 = x0, y1 = x1;
                    if (p.apply_rope) {
                        int i = ((qc0 + c) % D) / 2;
                        float cos_angle = isq ? cq[lr][i] : ck[lr][i];
                        float sin_angle = isq ? sq[lr][i] : sk[lr][i];
                        y0 = x0 * cos_angle - x1 * sin_angle;
                        y1 = x0 * sin_angle + x1 * cos_angle;
                    }
                    if (isq) { Qs[lr][2 * pr] = y0; Qs[lr][2 * pr + 1] = y1; }
                    else { Ks[lr][2 * pr] = y0; Ks[lr][2 * pr + 1] = y1; }
                }
                __syncthreads();
#pragma unroll
                for (int kk = 0; kk < AF_BK; ++kk) {
                    float a = Qs[r][kk];
#pragma unroll
                    for (int j = 0; j < 4; ++j) s[j] = fmaf(a, Ks[cg + 16 * j][kk], s[j]);
                }
            }
            // scale (a separate fp32 multiply, as op_multiply does) and mask
            bool ok[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                s[j] = s[j] * p.scale;
                ok[j] = (j0 + cg + 16 * j) <= row_last;
            }
            if (pass == 0) {
                float tm = -INFINITY;
#pragma unroll
                for (int j = 0; j < 4; ++j) if (ok[j]) tm = fmaxf(tm, s[j]);
#pragma unroll
                for (int o = 1; o < 16; o <<= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
                float m_new = fmaxf(m_run, tm);
                float ts = 0.0f;
#pragma unroll
                for (int j = 0; j < 4; ++j) if (ok[j]) ts += expf(s[j] - m_new);
#pragma unroll
                for (int o = 1; o < 16; o <<= 1) ts += __shfl_xor_sync(0xffffffffu, ts, o);
                if (m_new > -INFINITY) {
                    l_run = l_run * expf(m_run - m_new) + ts;
                    m_run = m_new;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) Ps[r][cg + 16 * j] = ok[j] ? expf(s[j] - m_run) / l_run : 0.0f;
                __syncthreads();
                if (grow < p.S) {
                    int jmax = min(AF_BN, p.S - j0);
                    for (int jj = 0; jj < jmax; ++jj) {
                        float pv = Ps[r][jj];
                        const float* vrow = p.v + (int64_t)(j0 + jj) * p.v_rs;
#pragma unroll
                        for (int oc = 0; oc < AF_MAXOUT; ++oc) {
                            int c = cg + 16 * oc;
                            if (c < Wo) acc[oc] = fmaf(pv, vrow[(vc0 + c) * p.v_cs], acc[oc]);
                        }
                    }
                }
            }
        }
    }
    if (grow >= p.S) return;
#pragma unroll
    for (int oc = 0; oc < AF_MAXOUT; ++oc) {
        int c = cg + 16 * oc;
        if (c >= Wo) continue;
        if (collapsed) {
            int g = c / D, d = c % D;
            for (int rep = 0; rep < n_rep; ++rep)
                p.out[grow * p.o_rs + ((g * n_rep + rep) * D + d) * p.o_cs] = acc[oc];
        } else {
            p.out[grow * p.o_rs + (prob * D + c) * p.o_cs] = acc[oc];
        }
    }
}

}  // namespace bn

using namespace bn;

extern "C" int bn_mm_f32(const float* A, int64_t a_rs, int64_t a_cs, const float* B, int64_t b_rs, int64_t b_cs,
                         float* C, int64_t c_rs, int64_t c_cs, int M, int K, int N, bn_stream_t stream) {
    if (!A || !B || !C) return fail(BN_ERR_INVALID_ARG, "bn_mm_f32: null pointer");
    if (M < 0 || K < 0 || N < 0) return fail(BN_ERR_INVALID_ARG, "bn_mm_f32: negative size");
    if (int rc = require_sm100()) return rc;
    if (M == 0 || N == 0) return BN_OK;
    dim3 grid(ceil_div(N, MM_T), ceil_div(M, MM_T));
    if (grid.y > 65535) return fail(BN_ERR_UNSUPPORTED, "bn_mm_f32: M=%d too large", M);
    mm_f32_kernel<<<grid, 256, 0, as_stream(stream)>>>(A, a_rs, a_cs, B, b_rs, b_cs, C, c_rs, c_cs, M, K, N);
    return launch_status("bn_mm_f32");
}

extern "C" int bn_rope_f32(const float* x, int64_t x_rs, int64_t x_cs, float* y, int64_t y_rs, int64_t y_cs,
                           int rows, int cols, int head_dim, float theta, int position_offset,
                           bn_stream_t stream) {
    if (!x || !y) return fail(BN_ERR_INVALID_ARG, "bn_rope_f32: null pointer");
    if (rows < 0 || cols < 0 || head_dim <= 0 || head_dim % 2)
        return fail(BN_ERR_INVALID_ARG, "bn_rope_f32: bad shape rows=%d cols=%d head_dim=%d", rows, cols, head_dim);
    if (cols % head_dim != 0)
        return fail(BN_ERR_INVALID_ARG, "RoPE: hidden_dim must be divisible by head_dim");  // op_rope.cuh:115-117
    if (int rc = require_sm100()) return rc;
    int64_t n = (int64_t)rows * (cols / 2);
    if (n == 0) return BN_OK;
    rope_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(x, x_rs, x_cs, y, y_rs, y_cs, rows,
                                                                               cols, head_dim, theta,
                                                                               position_offset);
    return launch_status("bn_rope_f32");
}

extern "C" int bn_attn_prefill_f32(const float* q, int64_t q_rs, int64_t q_cs, const float* k, int64_t k_rs,
                                   int64_t k_cs, const float* v, int64_t v_rs, int64_t v_cs, float* out,
                                   int64_t o_rs, int64_t o_cs, int S, int Hq, int Hkv, int D, float scale,
                                   float theta, int position_offset, int causal, int heads_mode, int apply_rope,
                                   bn_stream_t stream) {
    if (!q || !k || !v || !out) return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_f32: null pointer");
    if (S < 0 || Hq <= 0 || Hkv <= 0 || D <= 0)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_f32: bad shape S=%d Hq=%d Hkv=%d D=%d", S, Hq, Hkv, D);
    if (Hq % Hkv != 0) return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_f32: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
    if (heads_mode != BN_HEADS_COLLAPSED && heads_mode != BN_HEADS_PER_HEAD)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_f32: heads_mode=%d", heads_mode);
    if (D % 2 || D > 2 * AF_MAXHALF)
        return fail(BN_ERR_UNSUPPORTED, "bn_attn_prefill_f32: head_dim=%d (even, <= %d supported)", D, 2 * AF_MAXHALF);
    int Wo = heads_mode == BN_HEADS_COLLAPSED ? Hkv * D : D;
    if (Wo > 16 * AF_MAXOUT)
        return fail(BN_ERR_UNSUPPORTED, "bn_attn_prefill_f32: Hkv*D=%d (<= %d supported)", Wo, 16 * AF_MAXOUT);
    if (int rc = require_sm100()) return rc;
    if (S == 0) return BN_OK;
    AttnF32Params p{q, k, v, out, q_rs, q_cs, k_rs, k_cs, v_rs, v_cs, o_rs, o_cs, S, Hq, Hkv, D,
                    scale, theta, position_offset, causal, heads_mode, apply_rope};
    dim3 grid(ceil_div(S, AF_BM), heads_mode == BN_HEADS_COLLAPSED ? 1 : Hq);
    attn_f32_kernel<<<grid, 256, 0, as_stream(stream)>>>(p);
    return launch_status("bn_attn_prefill_f32");
}

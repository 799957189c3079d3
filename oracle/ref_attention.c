/*
 * CPU restatement (plain C) of BareNet's grouped-query attention operators.
 *
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA path and the timed CPU
 * baseline.  Nothing that ships links or loads this file.
 *
 * Parity status: the reference holds no golden vectors for this path; this
 * restatement is pinned against outputs of the reference's own CUDA operators
 * run on a B200 (fixtures under tests/golden/).
 *
 * The reference's operators are fp32 SIMT kernels whose arithmetic order is
 * fully determined by their source, so each function below keeps that order:
 *   - GEMM: one fused-multiply-add chain per output element, k ascending
 *     (src/ops/op_mm_optimized.cuh:35-62 and src/ops/op_mm.cuh:23-36; nvcc
 *     contracts `sum += a*b` into an FMA, hence fmaf here).
 *   - RoPE: src/ops/op_rope.cuh:55-99.
 *   - causal softmax: src/ops/op_softmax.cuh:76-151 (256 strided partials,
 *     then a pairwise tree).
 *   - layer composition: mygrad/llama/llama_layers.py:140-188.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off -mfma -fopenmp).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define REF_EXPORT __attribute__((visibility("default")))

REF_EXPORT int ref_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

REF_EXPORT void ref_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* freq_i = 1.0 / powf(theta, (float)(2 i) / head_dim)   (op_rope.cuh:82) */
REF_EXPORT void ref_rope_inv_freq(int head_dim, float theta, float* inv_freq) {
    for (int i = 0; i < head_dim / 2; ++i) {
        float e = (float)(2 * i) / head_dim;
        inv_freq[i] = (float)(1.0 / powf(theta, e));
    }
}

/* out[r][c] for a dense (rows, cols) matrix; row r is at position
 * r + position_offset.  inv_freq may be NULL (computed as above) or a table of
 * head_dim/2 floats.                                   (op_rope.cuh:55-99) */
REF_EXPORT void ref_rope_f32(const float* x, int rows, int cols, int head_dim, float theta,
                             int position_offset, const float* inv_freq, float* out) {
    int half = head_dim / 2;
    float* tab = (float*)malloc(sizeof(float) * (size_t)half);
    if (inv_freq) memcpy(tab, inv_freq, sizeof(float) * (size_t)half);
    else ref_rope_inv_freq(head_dim, theta, tab);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        int position = r + position_offset;
        for (int c0 = 0; c0 < cols; c0 += 2) {
            int pair = (c0 % head_dim) / 2;
            float angle = position * tab[pair];
            float cs = cosf(angle), sn = sinf(angle);
            float x0 = x[(size_t)r * cols + c0], x1 = x[(size_t)r * cols + c0 + 1];
            /* nvcc contracts a*b - c*d into fma(a, b, -(c*d)) style chains; the
             * two roundings differ by <= 1 ulp of the product, far inside every
             * gate used here, so the plain expression is kept. */
            out[(size_t)r * cols + c0] = x0 * cs - x1 * sn;
            out[(size_t)r * cols + c0 + 1] = x0 * sn + x1 * cs;
        }
    }
    free(tab);
}

/* C (M,N) = A (M,K) * B (K,N); element strides given so that B may be a
 * transposed view, as in `query @ key.T` (llama_layers.py:174).
 * One FMA chain per output, k ascending.               (op_mm*.cuh) */
REF_EXPORT void ref_mm_f32(const float* A, long a_rs, long a_cs, const float* B, long b_rs, long b_cs,
                           float* C, int M, int K, int N) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < M; ++i) {
        for (int j = 0; j < N; ++j) {
            float sum = 0.0f;
            const float* a = A + (size_t)i * a_rs;
            const float* b = B + (size_t)j * b_cs;
            for (int k = 0; k < K; ++k) sum = fmaf(a[(size_t)k * a_cs], b[(size_t)k * b_rs], sum);
            C[(size_t)i * N + j] = sum;
        }
    }
}

/* Row softmax with the reference's reduction shape: thread t of 256 handles
 * columns t, t+256, ...; max and sum are tree-reduced with halving strides.
 * causal: column j valid iff j <= row + seq_offset; masked -> 0.
 *                                                     (op_softmax.cuh:8-151) */
REF_EXPORT void ref_softmax_f32(const float* in, int rows, int cols, int causal, int seq_offset, float* out) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        float part[256];
        const float* x = in + (size_t)r * cols;
        float* y = out + (size_t)r * cols;
        int qpos = causal ? r + seq_offset : cols;
        for (int t = 0; t < 256; ++t) {
            float m = -INFINITY;
            for (int i = t; i < cols; i += 256)
                if (i <= qpos && x[i] > m) m = x[i];
            part[t] = m;
        }
        for (int s = 128; s > 0; s >>= 1)
            for (int t = 0; t < s; ++t)
                if (part[t + s] > part[t]) part[t] = part[t + s];
        float mx = part[0];
        for (int t = 0; t < 256; ++t) {
            float acc = 0.0f;
            for (int i = t; i < cols; i += 256) {
                if (i <= qpos) { float e = expf(x[i] - mx); y[i] = e; acc += e; }
                else y[i] = 0.0f;
            }
            part[t] = acc;
        }
        for (int s = 128; s > 0; s >>= 1)
            for (int t = 0; t < s; ++t) part[t] += part[t + s];
        float sum = part[0];
        for (int i = 0; i < cols; ++i)
            if (i <= qpos) y[i] = y[i] / sum;
    }
}

/* dst head kv_head*n_rep+rep <- src head kv_head  (llama_layers.py:126-136) */
static void repeat_kv(const float* kv, int rows, int n_kv, int n_rep, int D, float* out) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r)
        for (int g = 0; g < n_kv; ++g)
            for (int rep = 0; rep < n_rep; ++rep)
                memcpy(out + ((size_t)r * n_kv * n_rep + (size_t)g * n_rep + rep) * D,
                       kv + ((size_t)r * n_kv + g) * D, sizeof(float) * (size_t)D);
}

/* The attention core exactly as the layer composes it (llama_layers.py:161-183):
 * rope(q), rope(k), repeat, scores = q @ k^T over the FULL Hq*D width, * scale,
 * one (S,S) softmax, probs @ v.  q (S, Hq*D), k,v (S, Hkv*D), out (S, Hq*D). */
REF_EXPORT int ref_attention_collapsed_f32(const float* q, const float* k, const float* v, int S, int Hq,
                                           int Hkv, int D, float theta, int position_offset, int causal,
                                           const float* inv_freq, float* out) {
    int Wq = Hq * D, Wk = Hkv * D, n_rep = Hq / Hkv;
    float scale = (float)(1.0 / sqrt((double)D));
    float* qr = (float*)malloc(sizeof(float) * (size_t)S * Wq);
    float* kr = (float*)malloc(sizeof(float) * (size_t)S * Wk);
    float* kk = (float*)malloc(sizeof(float) * (size_t)S * Wq);
    float* vv = (float*)malloc(sizeof(float) * (size_t)S * Wq);
    float* sc = (float*)malloc(sizeof(float) * (size_t)S * S);
    float* pr = (float*)malloc(sizeof(float) * (size_t)S * S);
    if (!qr || !kr || !kk || !vv || !sc || !pr) return 1;
    ref_rope_f32(q, S, Wq, D, theta, position_offset, inv_freq, qr);
    ref_rope_f32(k, S, Wk, D, theta, position_offset, inv_freq, kr);
    repeat_kv(kr, S, Hkv, n_rep, D, kk);
    repeat_kv(v, S, Hkv, n_rep, D, vv);
    ref_mm_f32(qr, Wq, 1, kk, 1, Wq, sc, S, Wq, S); /* B = kk^T view: b_rs=1, b_cs=Wq */
    for (size_t i = 0; i < (size_t)S * S; ++i) sc[i] = sc[i] * scale;
    ref_softmax_f32(sc, S, S, causal, position_offset, pr);
    ref_mm_f32(pr, S, 1, vv, Wq, 1, out, S, S, Wq);
    free(qr); free(kr); free(kk); free(vv); free(sc); free(pr);
    return 0;
}

/* GroupedQueryAttention.__call__ (llama_layers.py:140-188). Weights (in,out). */
REF_EXPORT int ref_gqa_layer_f32(const float* x, const float* wq, const float* wk, const float* wv,
                                 const float* wo, int S, int hidden, int Hq, int Hkv, int D, float theta,
                                 int position_offset, int causal, const float* inv_freq, float* out) {
    int Wq = Hq * D, Wk = Hkv * D;
    float* q = (float*)malloc(sizeof(float) * (size_t)S * Wq);
    float* k = (float*)malloc(sizeof(float) * (size_t)S * Wk);
    float* v = (float*)malloc(sizeof(float) * (size_t)S * Wk);
    float* a = (float*)malloc(sizeof(float) * (size_t)S * Wq);
    if (!q || !k || !v || !a) return 1;
    ref_mm_f32(x, hidden, 1, wq, Wq, 1, q, S, hidden, Wq);
    ref_mm_f32(x, hidden, 1, wk, Wk, 1, k, S, hidden, Wk);
    ref_mm_f32(x, hidden, 1, wv, Wk, 1, v, S, hidden, Wk);
    int rc = ref_attention_collapsed_f32(q, k, v, S, Hq, Hkv, D, theta, position_offset, causal, inv_freq, a);
    if (rc == 0) ref_mm_f32(a, Wq, 1, wo, hidden, 1, out, S, Wq, hidden);
    free(q); free(k); free(v); free(a);
    return rc;
}

/* Per-head grouped-query attention: the same operators (RoPE, q k^T, *scale,
 * causal softmax, p v) applied independently to every D-wide head, query head h
 * reading KV head h / n_rep.  Inputs are fp32 arrays (for the bf16 workloads
 * they hold bf16-exact values).  q (B,S,Hq,D), k,v (B,S,Hkv,D), out (B,S,Hq,D).
 * Work is done only for batches [b0,b1) and query heads [h0,h1) so that a
 * bounded sample of a big workload can be timed.  round_bf16 != 0 rounds the
 * rotated q,k to bf16 as a tensor-core path does. */
static inline float bf16_round(float x) {
    uint32_t u; memcpy(&u, &x, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    u &= 0xFFFF0000u;
    float y; memcpy(&y, &u, 4);
    return y;
}

REF_EXPORT int ref_attention_per_head_f32(const float* q, const float* k, const float* v, int B, int S, int Hq,
                                          int Hkv, int D, float theta, int position_offset, int causal,
                                          int round_bf16, const float* inv_freq, int b0, int b1, int h0, int h1,
                                          float* out) {
    (void)B;
    int n_rep = Hq / Hkv, half = D / 2;
    float scale = (float)(1.0 / sqrt((double)D));
    float* tab = (float*)malloc(sizeof(float) * (size_t)half);
    float* cs = (float*)malloc(sizeof(float) * (size_t)S * half);
    float* sn = (float*)malloc(sizeof(float) * (size_t)S * half);
    if (!tab || !cs || !sn) return 1;
    if (inv_freq) memcpy(tab, inv_freq, sizeof(float) * (size_t)half);
    else ref_rope_inv_freq(D, theta, tab);
    for (int r = 0; r < S; ++r)
        for (int i = 0; i < half; ++i) {
            float angle = (r + position_offset) * tab[i];
            cs[(size_t)r * half + i] = cosf(angle);
            sn[(size_t)r * half + i] = sinf(angle);
        }
    int err = 0;
    for (int b = b0; b < b1; ++b) {
        for (int h = h0; h < h1; ++h) {
            int g = h / n_rep;
            float* qr = (float*)malloc(sizeof(float) * (size_t)S * D);
            float* kr = (float*)malloc(sizeof(float) * (size_t)S * D);
            if (!qr || !kr) { err = 1; free(qr); free(kr); break; }
#pragma omp parallel for schedule(static)
            for (int r = 0; r < S; ++r) {
                const float* qs = q + (((size_t)b * S + r) * Hq + h) * D;
                const float* ks = k + (((size_t)b * S + r) * Hkv + g) * D;
                for (int i = 0; i < half; ++i) {
                    float c = cs[(size_t)r * half + i], s = sn[(size_t)r * half + i];
                    float a0 = qs[2 * i] * c - qs[2 * i + 1] * s, a1 = qs[2 * i] * s + qs[2 * i + 1] * c;
                    float b0_ = ks[2 * i] * c - ks[2 * i + 1] * s, b1_ = ks[2 * i] * s + ks[2 * i + 1] * c;
                    if (round_bf16) { a0 = bf16_round(a0); a1 = bf16_round(a1); b0_ = bf16_round(b0_); b1_ = bf16_round(b1_); }
                    qr[(size_t)r * D + 2 * i] = a0; qr[(size_t)r * D + 2 * i + 1] = a1;
                    kr[(size_t)r * D + 2 * i] = b0_; kr[(size_t)r * D + 2 * i + 1] = b1_;
                }
            }
#pragma omp parallel
            {
                float* sc = (float*)malloc(sizeof(float) * (size_t)S);
#pragma omp for schedule(dynamic, 8)
                for (int r = 0; r < S; ++r) {
                    int last = causal ? r + position_offset : S - 1;
                    if (last > S - 1) last = S - 1;
                    float mx = -INFINITY;
                    for (int j = 0; j <= last; ++j) {
                        float sum = 0.0f;
                        for (int d = 0; d < D; ++d) sum = fmaf(qr[(size_t)r * D + d], kr[(size_t)j * D + d], sum);
                        sum *= scale;
                        sc[j] = sum;
                        if (sum > mx) mx = sum;
                    }
                    float den = 0.0f;
                    for (int j = 0; j <= last; ++j) { sc[j] = expf(sc[j] - mx); den += sc[j]; }
                    float* o = out + (((size_t)b * S + r) * Hq + h) * D;
                    for (int d = 0; d < D; ++d) o[d] = 0.0f;
                    for (int j = 0; j <= last; ++j) {
                        float p = sc[j] / den;
                        const float* vs = v + (((size_t)b * S + j) * Hkv + g) * D;
                        for (int d = 0; d < D; ++d) o[d] = fmaf(p, vs[d], o[d]);
                    }
                }
                free(sc);
            }
            free(qr); free(kr);
        }
        if (err) break;
    }
    free(tab); free(cs); free(sn);
    return err;
}

/* Single-token decode over a paged cache: the last row of a per-head prefill
 * over the cached tokens (decode semantics: llama_model.py:136-144).
 * pool: bf16 bit patterns (num_pages, Hkv, 2, 16, D); q (B, Hq, D) fp32 values
 * already rotated; out (B, Hq, D); lse (B, Hq) natural log (may be NULL).
 * Only sequences [s0, s1) are processed. */
static inline float bf16_bits_to_float(uint16_t b) {
    uint32_t u = ((uint32_t)b) << 16; float y; memcpy(&y, &u, 4); return y;
}

REF_EXPORT int ref_decode_paged_f32(const float* q, const uint16_t* pool, const int32_t* page_table,
                                    int max_pages, const int32_t* seq_lens, int Hq, int Hkv, int D,
                                    int s0, int s1, float* out, float* lse) {
    int n_rep = Hq / Hkv;
    float scale = (float)(1.0 / sqrt((double)D));
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (int b = s0; b < s1; ++b) {
        for (int h = 0; h < Hq; ++h) {
            int L = seq_lens[b], g = h / n_rep;
            float* o = out + ((size_t)b * Hq + h) * D;
            for (int d = 0; d < D; ++d) o[d] = 0.0f;
            if (L <= 0) { if (lse) lse[(size_t)b * Hq + h] = -INFINITY; continue; }
            float* sc = (float*)malloc(sizeof(float) * (size_t)L);
            const float* qv = q + ((size_t)b * Hq + h) * D;
            float mx = -INFINITY;
            for (int t = 0; t < L; ++t) {
                int page = page_table[(size_t)b * max_pages + t / 16];
                const uint16_t* kp = pool + ((((size_t)page * Hkv + g) * 2 + 0) * 16 + t % 16) * D;
                float sum = 0.0f;
                for (int d = 0; d < D; ++d) sum = fmaf(qv[d], bf16_bits_to_float(kp[d]), sum);
                sum *= scale; sc[t] = sum; if (sum > mx) mx = sum;
            }
            float den = 0.0f;
            for (int t = 0; t < L; ++t) { sc[t] = expf(sc[t] - mx); den += sc[t]; }
            for (int t = 0; t < L; ++t) {
                int page = page_table[(size_t)b * max_pages + t / 16];
                const uint16_t* vp = pool + ((((size_t)page * Hkv + g) * 2 + 1) * 16 + t % 16) * D;
                float p = sc[t] / den;
                for (int d = 0; d < D; ++d) o[d] = fmaf(p, bf16_bits_to_float(vp[d]), o[d]);
            }
            if (lse) lse[(size_t)b * Hq + h] = mx + logf(den);
            free(sc);
        }
    }
    return 0;
}

/* ---------------------------------------------------------------------------
 * RMSNorm, row-wise:  y = x / sqrt(mean(x^2) + eps) * w
 * Restates op_rmsnorm_kernel (src/ops/op_rmsnorm.cuh:8-53, launched with 256
 * threads per row, :134-157) in its own arithmetic order, so the result is the
 * reference's bit for bit:
 *   - thread t accumulates x[t], x[t+256], ... as a fused multiply-add chain
 *     (`sum_sq += val * val` contracts to FFMA under nvcc's defaults);
 *   - the 256 partial sums are reduced by the shared-memory tree
 *     sh[t] += sh[t + stride], stride = 128, 64, ..., 1;
 *   - mean = total / hidden (IEEE division), rms = sqrtf(mean + eps);
 *   - y = (x / rms) * w  (division first, then the weight).
 * `residual` (optional) is added to x first, in fp32, as the decoder layer's
 * `residual + hidden_states` does before the next norm (op_add,
 * mygrad/llama/llama_layers.py:279-283); the sum is returned in `sum_out`.
 * ------------------------------------------------------------------------- */
REF_EXPORT void ref_add_rmsnorm_f32(const float* x, const float* residual, const float* w, int rows, int hidden,
                                    float eps, float* sum_out, float* y) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const float* xr = x + (size_t)r * hidden;
        const float* rr = residual ? residual + (size_t)r * hidden : NULL;
        float* sr = sum_out ? sum_out + (size_t)r * hidden : NULL;
        float sh[256];
        for (int t = 0; t < 256; ++t) {
            float acc = 0.0f;
            for (int i = t; i < hidden; i += 256) {
                float v = rr ? xr[i] + rr[i] : xr[i];
                acc = fmaf(v, v, acc);
            }
            sh[t] = acc;
        }
        for (int stride = 128; stride > 0; stride >>= 1)
            for (int t = 0; t < stride; ++t) sh[t] += sh[t + stride];
        float mean_sq = sh[0] / (float)hidden;
        float rms = sqrtf(mean_sq + eps);
        for (int i = 0; i < hidden; ++i) {
            float v = rr ? xr[i] + rr[i] : xr[i];
            if (sr) sr[i] = v;
            y[(size_t)r * hidden + i] = (v / rms) * w[i];
        }
    }
}

REF_EXPORT void ref_rmsnorm_f32(const float* x, const float* w, int rows, int hidden, float eps, float* y) {
    ref_add_rmsnorm_f32(x, NULL, w, rows, hidden, eps, NULL, y);
}

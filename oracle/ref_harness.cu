/*
 * Driver around the reference's OWN CUDA operators, compiled from the header
 * files where they lie in the reference tree (never copied here); the built
 * library goes to oracle/_ref/ and is used only as a checker by the tests and
 * to generate tests/golden/ fixtures on a GPU.
 *
 * TEST INFRASTRUCTURE ONLY: nothing that ships links or loads this.
 *
 * Each entry point performs, on the reference's Tensor<float> type and op_*
 * launchers, the exact operator sequence of
 *   GroupedQueryAttention.__call__   (mygrad/llama/llama_layers.py:140-188)
 * i.e. op_mm, op_rope, the host-side head repeat, op_mm on a transposed view,
 * op_multiply(scalar), op_softmax(causal, seq_offset), op_mm, op_mm.
 *
 * All pointers are HOST pointers to dense row-major fp32.  Return 0 on
 * success, 1 on a thrown reference error (message via refgpu_last_error()).
 */
#include <cstring>
#include <string>
#include <vector>
#include <stdexcept>
#include <cuda_runtime.h>

#include "utils/tensor.cuh"
#include "ops/op_elemwise.cuh"
#include "ops/op_mm.cuh"
#include "ops/op_mm_optimized.cuh"
#include "ops/op_reduction.cuh"
#include "ops/op_rmsnorm.cuh"
#include "ops/op_rope.cuh"
#include "ops/op_softmax.cuh"

unsigned long long randgen_seed = 42;  // the symbol op_elemwise.cuh declares extern

static std::string g_err;

static Tensor<float> upload(const float* host, int h, int w) {
    Tensor<float> t(h, w, true);
    CUDA_OK(cudaMemcpy(t.rawp, host, sizeof(float) * (size_t)h * w, cudaMemcpyHostToDevice));
    return t;
}

static void download(const Tensor<float>& t, float* host) {
    CUDA_OK(cudaDeviceSynchronize());
    CUDA_OK(cudaMemcpy(host, t.rawp, sizeof(float) * (size_t)t.h * t.w, cudaMemcpyDeviceToHost));
}

// head repeat through the host, as both reference layers do it
// (llama_layers.py:105-138, llama_layers.hpp:131-175)
static Tensor<float> repeat_heads(const Tensor<float>& kv, int n_rep, int head_dim) {
    if (n_rep == 1) return kv;
    int rows = kv.h, n_kv = kv.w / head_dim;
    std::vector<float> src((size_t)rows * kv.w), dst((size_t)rows * kv.w * n_rep);
    CUDA_OK(cudaDeviceSynchronize());
    CUDA_OK(cudaMemcpy(src.data(), kv.rawp, sizeof(float) * src.size(), cudaMemcpyDeviceToHost));
    for (int r = 0; r < rows; ++r)
        for (int g = 0; g < n_kv; ++g)
            for (int rep = 0; rep < n_rep; ++rep)
                std::memcpy(&dst[((size_t)r * n_kv * n_rep + (size_t)g * n_rep + rep) * head_dim],
                            &src[((size_t)r * n_kv + g) * head_dim], sizeof(float) * head_dim);
    return upload(dst.data(), rows, kv.w * n_rep);
}

static Tensor<float> attention_core(const Tensor<float>& q_in, const Tensor<float>& k_in, const Tensor<float>& v_in,
                                    int Hq, int Hkv, int D, float theta, int position_offset, int causal,
                                    int apply_rope) {
    int S = q_in.h;
    Tensor<float> q = q_in, k = k_in;
    if (apply_rope) {
        q = Tensor<float>(S, q_in.w, true);
        k = Tensor<float>(S, k_in.w, true);
        op_rope<float>(q_in, q, position_offset, D, theta);
        op_rope<float>(k_in, k, position_offset, D, theta);
    }
    int n_rep = Hq / Hkv;
    Tensor<float> kk = repeat_heads(k, n_rep, D);
    Tensor<float> vv = repeat_heads(v_in, n_rep, D);
    Tensor<float> scores(S, S, true);
    op_mm<float>(q, kk.transpose(), scores);
    Tensor<float> scaled(S, S, true);
    float scale = (float)(1.0 / sqrt((double)D));  // np.float64 1/np.sqrt(D) cast to T at the binding
    op_multiply<float>(scores, scale, scaled);
    Tensor<float> probs(S, S, true);
    op_softmax<float>(scaled, probs, causal != 0, position_offset);
    Tensor<float> out(S, q_in.w, true);
    op_mm<float>(probs, vv, out);
    return out;
}

__global__ void dump_inv_freq_kernel(float* out, int head_dim, float theta) {
    int i = threadIdx.x;
    if (i < head_dim / 2) out[i] = 1.0 / pow(theta, (float)(2 * i) / head_dim);  // op_rope.cuh:82
}

extern "C" {

const char* refgpu_last_error() { return g_err.c_str(); }

int refgpu_inv_freq(int head_dim, float theta, float* out) {
    try {
        float* d;
        CUDA_OK(cudaMalloc(&d, sizeof(float) * head_dim));
        dump_inv_freq_kernel<<<1, 128>>>(d, head_dim, theta);
        CUDA_OK(cudaDeviceSynchronize());
        CUDA_OK(cudaMemcpy(out, d, sizeof(float) * (head_dim / 2), cudaMemcpyDeviceToHost));
        cudaFree(d);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return 1; }
}

// op_argmax (src/ops/op_reduction.cuh:196-210): per-row index of the first maximum, (rows, 1) uint32
int refgpu_argmax(const float* x, int rows, int cols, unsigned int* out) {
    try {
        Tensor<float> in = upload(x, rows, cols);
        Tensor<unsigned int> idx(rows, 1, true);
        op_argmax<float, unsigned int>(in, idx);
        CUDA_OK(cudaDeviceSynchronize());
        CUDA_OK(cudaMemcpy(out, idx.rawp, sizeof(unsigned int) * rows, cudaMemcpyDeviceToHost));
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return 1; }
}

// op_rmsnorm (src/ops/op_rmsnorm.cuh:134-157): weight is a (1, hidden) tensor
int refgpu_rmsnorm(const float* x, const float* w, int rows, int hidden, float eps, float* out) {
    try {
        Tensor<float> in = upload(x, rows, hidden), wt = upload(w, 1, hidden), o(rows, hidden, true);
        op_rmsnorm<float>(in, wt, o, eps);
        download(o, out);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return 1; }
}

int refgpu_rope(const float* x, int rows, int cols, int head_dim, float theta, int position_offset, float* out) {
    try {
        Tensor<float> in = upload(x, rows, cols), o(rows, cols, true);
        op_rope<float>(in, o, position_offset, head_dim, theta);
        download(o, out);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return 1; }
}

int refgpu_attention_core(const float* q, const float* k, const float* v, int S, int Hq, int Hkv, int D,
                          float theta, int position_offset, int causal, int apply_rope, float* out) {
    try {
        Tensor<float> tq = upload(q, S, Hq * D), tk = upload(k, S, Hkv * D), tv = upload(v, S, Hkv * D);
        Tensor<float> o = attention_core(tq, tk, tv, Hq, Hkv, D, theta, position_offset, causal, apply_rope);
        download(o, out);
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return 1; }
}

// whole layer; if time_ms != NULL the forward is repeated `iters` times after
// `warmup` runs and the mean CUDA-event time per forward is stored there.
int refgpu_gqa_layer(const float* x, const float* wq, const float* wk, const float* wv, const float* wo,
                     int S, int hidden, int Hq, int Hkv, int D, float theta, int position_offset, int causal,
                     float* out, int warmup, int iters, float* time_ms) {
    try {
        Tensor<float> tx = upload(x, S, hidden);
        Tensor<float> twq = upload(wq, hidden, Hq * D), twk = upload(wk, hidden, Hkv * D);
        Tensor<float> twv = upload(wv, hidden, Hkv * D), two = upload(wo, Hq * D, hidden);
        auto forward = [&]() {
            Tensor<float> q(S, Hq * D, true), k(S, Hkv * D, true), v(S, Hkv * D, true);
            op_mm<float>(tx, twq, q);
            op_mm<float>(tx, twk, k);
            op_mm<float>(tx, twv, v);
            Tensor<float> a = attention_core(q, k, v, Hq, Hkv, D, theta, position_offset, causal, 1);
            Tensor<float> o(S, hidden, true);
            op_mm<float>(a, two, o);
            return o;
        };
        Tensor<float> o = forward();
        download(o, out);
        if (time_ms) {
            for (int i = 0; i < warmup; ++i) forward();
            cudaEvent_t e0, e1;
            CUDA_OK(cudaEventCreate(&e0)); CUDA_OK(cudaEventCreate(&e1));
            CUDA_OK(cudaDeviceSynchronize());
            CUDA_OK(cudaEventRecord(e0));
            for (int i = 0; i < iters; ++i) forward();
            CUDA_OK(cudaEventRecord(e1));
            CUDA_OK(cudaEventSynchronize(e1));
            float ms = 0;
            CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
            *time_ms = ms / (iters > 0 ? iters : 1);
            cudaEventDestroy(e0); cudaEventDestroy(e1);
        }
        return 0;
    } catch (const std::exception& e) { g_err = e.what(); return 1; }
}

}  // extern "C"

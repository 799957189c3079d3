// bf16 prefill attention for sm_100a: RoPE on Q/K, causal Q K^T, online softmax
// and P V fused, per-head grouped-query attention.
//
// The math is the reference's operator sequence (rope -> q k^T -> *scale ->
// causal softmax -> p v; mygrad/llama/llama_layers.py:161-183 with
// src/ops/op_rope.cuh:55-99 and src/ops/op_softmax.cuh:76-151) applied per
// 64-wide head, query head h reading KV head h / (Hq/Hkv)
// (llama_layers.py:126-136), on bf16 operands with fp32 accumulation.
//
// Two launches:
//   1. rope_k_kernel: rotates K once into scratch (K is read by 8 query heads
//      x S/128 query tiles, so it is rotated once, not per use) and writes the
//      cos/sin table of the S positions.
//   2. prefill_kernel: one CTA per (batch, query head, 128-row query tile),
//      two CTAs resident per SM.
//        warps 0-3  softmax: one query row per thread (TMEM lane = row), so the
//                   row max / row sum need no cross-thread traffic; they also
//                   rotate the Q tile into swizzled shared memory (prologue)
//                   and write O (epilogue)
//        warp 4     TMA producer: K/V tiles of 128 keys through a 2-stage ring
//        warp 5     MMA issuer: tcgen05.mma, S = Q K^T (128x128x64) into TMEM,
//                   O += P V (128x64x128) with P read from TMEM
//      TMEM (256 columns): S fp32 [0,128) | O fp32 [128,192) | P bf16 [192,256)
//      Softmax works in base 2 with the scale folded into the exponent, masks
//      only tiles that touch the diagonal, skips tiles above it, and rescales O
//      only when the running maximum has grown by more than 2^8.
//   Every mbarrier wait is bounded; on expiry the kernel raises the error word
//   at the head of the scratch buffer, frees its TMEM and returns.
#include <math.h>

#include "common.cuh"
#include "ptx.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace bn {

using namespace ptx;

constexpr int PF_D = 64;
constexpr int PF_BM = 128;           // query rows per CTA
constexpr int PF_BN = 128;           // keys per tile
constexpr int PF_NSTAGE = 2;
constexpr int PF_TILE_BYTES = PF_BN * PF_D * 2;   // 16384
constexpr int PF_THREADS = 192;
constexpr int PF_SMEM_BYTES = 1024 + PF_TILE_BYTES * (1 + 2 * PF_NSTAGE);
constexpr uint32_t PF_TMEM_COLS = 256;
constexpr uint32_t PF_COL_S = 0, PF_COL_O = 128, PF_COL_P = 192;
constexpr float PF_LOG2E = 1.4426950408889634f;
constexpr float PF_LN2 = 0.6931471805599453f;
constexpr float PF_RESCALE_THRESHOLD = 8.0f;   // log2 units

struct PrefillWsLayout {
    size_t table, krot, total;
};

static PrefillWsLayout prefill_layout(int B, int S, int Hkv) {
    PrefillWsLayout L;
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    L.table = 256;                                               // after the header (error word)
    L.krot = L.table + up((size_t)S * (PF_D / 2) * sizeof(float2));
    L.total = L.krot + up((size_t)B * S * Hkv * PF_D * sizeof(__nv_bfloat16));
    return L;
}

// ---------------------------------------------------------------------------
// launch 1: K rotation + cos/sin table
// ---------------------------------------------------------------------------
__global__ void rope_k_kernel(const __nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ krot,
                              float2* __restrict__ table, int B, int S, int Hkv, float theta, int position_offset,
                              int* __restrict__ error_word) {
    const int s = blockIdx.x, b = blockIdx.y;
    if (s == 0 && b == 0 && threadIdx.x == 0) *error_word = 0;
    const int pairs = Hkv * (PF_D / 2);
    for (int e = threadIdx.x; e < pairs; e += blockDim.x) {
        const int i = e % (PF_D / 2);
        const float freq = rope_inv_freq(i, PF_D, theta);
        const float angle = (s + position_offset) * freq;
        const float cos_angle = cosf(angle), sin_angle = sinf(angle);
        if (b == 0 && e < PF_D / 2) table[(size_t)s * (PF_D / 2) + i] = make_float2(cos_angle, sin_angle);
        const size_t idx = ((size_t)b * S + s) * Hkv * PF_D + 2 * e;
        const uint32_t raw = *reinterpret_cast<const uint32_t*>(k + idx);
        const float x0 = bf16_lo(raw), x1 = bf16_hi(raw);
        const float y0 = x0 * cos_angle - x1 * sin_angle;
        const float y1 = x0 * sin_angle + x1 * cos_angle;
        *reinterpret_cast<uint32_t*>(krot + idx) = pack_bf16(y0, y1);
    }
}

// ---------------------------------------------------------------------------
// launch 2: the attention kernel
// ---------------------------------------------------------------------------
struct PrefillParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    float* lse;
    const float2* table;
    int* error_word;
    int B, S, Hq, Hkv, n_rep, n_qtiles, position_offset, causal;
    float scale_log2;
};

__global__ void __launch_bounds__(PF_THREADS, 2)
prefill_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
               const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_q, bar_s, bar_p, bar_o;
    __shared__ __align__(8) uint64_t bar_kfull[PF_NSTAGE], bar_vfull[PF_NSTAGE], bar_empty[PF_NSTAGE];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = smem0;
    const uint32_t sK = smem0 + PF_TILE_BYTES;                       // PF_NSTAGE tiles
    const uint32_t sV = smem0 + PF_TILE_BYTES * (1 + PF_NSTAGE);     // PF_NSTAGE tiles

    // work unit: heavy (late) query tiles first; the 8 query heads of a KV group are neighbours
    const int BH = p.B * p.Hq;
    const int qt = p.n_qtiles - 1 - (int)(blockIdx.x / BH);
    const int bh = blockIdx.x % BH;
    const int b = bh / p.Hq, h = bh % p.Hq, g = h / p.n_rep;
    const int i0 = qt * PF_BM;
    // number of key tiles this query tile needs
    int last_key = p.S - 1;
    if (p.causal) last_key = min(last_key, i0 + PF_BM - 1 + p.position_offset);
    const int n_tiles = last_key >= 0 ? last_key / PF_BN + 1 : 0;

    if (tid == 0) {
        mbar_init(smem_u32(&bar_q), 128);
        mbar_init(smem_u32(&bar_s), 1);
        mbar_init(smem_u32(&bar_p), 128);
        mbar_init(smem_u32(&bar_o), 1);
        for (int s = 0; s < PF_NSTAGE; ++s) {
            mbar_init(smem_u32(&bar_kfull[s]), 1);
            mbar_init(smem_u32(&bar_vfull[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        s_abort = 0;
        fence_mbar_init();
    }
    if (warp == 5) {
        tc::tmem_alloc(smem_u32(&s_tmem_base), PF_TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = s_tmem_base;

    if (warp == 4) {
        // ---------------------------------------------------------- TMA producer
        if (lane == 0) {
            prefetch_tensormap(&tmap_k);
            prefetch_tensormap(&tmap_v);
            int stage = 0;
            uint32_t phase = 0;
            for (int j = 0; j < n_tiles; ++j) {
                if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &s_abort)) break;
                mbar_arrive_expect_tx(smem_u32(&bar_kfull[stage]), PF_TILE_BYTES);
                tma_load_4d(sK + stage * PF_TILE_BYTES, &tmap_k, 0, g, j * PF_BN, b, smem_u32(&bar_kfull[stage]));
                mbar_arrive_expect_tx(smem_u32(&bar_vfull[stage]), PF_TILE_BYTES);
                tma_load_4d(sV + stage * PF_TILE_BYTES, &tmap_v, 0, g, j * PF_BN, b, smem_u32(&bar_vfull[stage]));
                if (++stage == PF_NSTAGE) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t IDESC_QK = tc::idesc_bf16(PF_BM, PF_BN, 0);
        constexpr uint32_t IDESC_PV = tc::idesc_bf16(PF_BM, PF_D, 1);
        bool ok = mbar_wait(smem_u32(&bar_q), 0, &s_abort);
        int stage = 0;
        uint32_t phase = 0;
        // S_0 = Q K_0^T
        if (ok && n_tiles > 0) {
            ok = mbar_wait(smem_u32(&bar_kfull[0]), 0, &s_abort);
            if (ok && lane == 0) {
                tc::fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < PF_D / 16; ++kk)
                    tc::mma_ss(tmem + PF_COL_S, tc::smem_desc_sw128(sQ + kk * 32), tc::smem_desc_sw128(sK + kk * 32),
                               IDESC_QK, kk > 0);
                tc::commit(smem_u32(&bar_s));
            }
            __syncwarp();
        }
        for (int j = 0; ok && j < n_tiles; ++j) {
            // O += P_j V_j once the softmax warps have written P_j
            ok = mbar_wait(smem_u32(&bar_p), j & 1, &s_abort) && mbar_wait(smem_u32(&bar_vfull[stage]), phase, &s_abort);
            if (!ok) break;
            if (lane == 0) {
                tc::fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < PF_BN / 16; ++kk)
                    tc::mma_ts(tmem + PF_COL_O, tmem + PF_COL_P + kk * 8,
                               tc::smem_desc_sw128(sV + stage * PF_TILE_BYTES + kk * 2048), IDESC_PV, (j > 0) || (kk > 0));
                tc::commit(smem_u32(&bar_empty[stage]));      // K_j / V_j may be overwritten
                if (j == n_tiles - 1) tc::commit(smem_u32(&bar_o));
            }
            __syncwarp();
            if (++stage == PF_NSTAGE) { stage = 0; phase ^= 1u; }
            if (j + 1 < n_tiles) {
                // S_{j+1} = Q K_{j+1}^T; the S columns are free because P_j has been written
                ok = mbar_wait(smem_u32(&bar_kfull[stage]), phase, &s_abort);
                if (!ok) break;
                if (lane == 0) {
                    tc::fence_after_sync();
#pragma unroll
                    for (int kk = 0; kk < PF_D / 16; ++kk)
                        tc::mma_ss(tmem + PF_COL_S, tc::smem_desc_sw128(sQ + kk * 32),
                                   tc::smem_desc_sw128(sK + stage * PF_TILE_BYTES + kk * 32), IDESC_QK, kk > 0);
                    tc::commit(smem_u32(&bar_s));
                }
                __syncwarp();
            }
        }
    } else {
        // ------------------------------------------------ softmax warps (0..3)
        const int row = tid;                      // TMEM lane = query row inside the tile
        const int gi = i0 + row;                  // query row inside the sequence
        const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;

        // prologue: rotate the Q row and store it, 128-byte-swizzled, K-major
        {
            uint4 qv[8];
            const bool valid = gi < p.S;
            const uint4* src = reinterpret_cast<const uint4*>(p.q + (((size_t)b * p.S + (valid ? gi : 0)) * p.Hq + h) * PF_D);
            const float4* tab = reinterpret_cast<const float4*>(p.table + (size_t)(valid ? gi : 0) * (PF_D / 2));
#pragma unroll
            for (int c = 0; c < 8; ++c) qv[c] = valid ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint32_t w[4] = {qv[c].x, qv[c].y, qv[c].z, qv[c].w};
#pragma unroll
                for (int e = 0; e < 4; e += 2) {
                    const float4 cs = __ldg(tab + c * 2 + e / 2);   // (cos, sin) of pairs 4c+e, 4c+e+1
                    float x0 = bf16_lo(w[e]), x1 = bf16_hi(w[e]);
                    w[e] = pack_bf16(x0 * cs.x - x1 * cs.y, x0 * cs.y + x1 * cs.x);
                    x0 = bf16_lo(w[e + 1]); x1 = bf16_hi(w[e + 1]);
                    w[e + 1] = pack_bf16(x0 * cs.z - x1 * cs.w, x0 * cs.w + x1 * cs.z);
                }
                const uint32_t dst = sQ + row * 128 + ((c ^ (row & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                             : "memory");
            }
            fence_proxy_async_smem();
            mbar_arrive(smem_u32(&bar_q));
        }

        float m_ref = -INFINITY;   // exponent reference, raw score units
        float l_run = 0.f;
        bool ok = true;
        const int row_last = p.causal ? min(p.S - 1, gi + p.position_offset) : p.S - 1;   // last valid key of this row

        for (int j = 0; j < n_tiles; ++j) {
            ok = mbar_wait(smem_u32(&bar_s), j & 1, &s_abort);
            if (!ok) break;
            tc::fence_after_sync();
            const int j0 = j * PF_BN;
            // does any row of the tile need masking in this key tile?
            const bool need_mask = (j0 + PF_BN - 1) > (p.causal ? min(p.S - 1, i0 + p.position_offset) : p.S - 1);

            // pass 1: row maximum
            float tmax = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tc::ld32(tmem + lane_base + PF_COL_S + c * 32, r);
                tc::wait_ld();
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (j0 + c * 32 + i <= row_last) tmax = fmaxf(tmax, __uint_as_float(r[i]));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) tmax = fmaxf(tmax, __uint_as_float(r[i]));
                }
            }
            const float m_new = fmaxf(m_ref, tmax);
            // rescale O only when the maximum moved far; the decision is per warp because the
            // TMEM loads and stores below are warp-collective
            const bool grow = (m_new - m_ref) * p.scale_log2 > PF_RESCALE_THRESHOLD;   // also true when m_ref = -inf
            if (__any_sync(0xffffffffu, grow)) {
                const float m_upd = m_new == -INFINITY ? m_ref : m_new;
                if (j > 0) {
                    const float alpha = m_ref == -INFINITY ? 0.f : ex2((m_ref - m_upd) * p.scale_log2);
                    l_run *= alpha;
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint32_t r[32];
                        tc::ld32(tmem + lane_base + PF_COL_O + c * 32, r);
                        tc::wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tc::st32(tmem + lane_base + PF_COL_O + c * 32, r);
                    }
                }
                m_ref = m_upd;
            }
            const float mneg = m_ref == -INFINITY ? 0.f : -m_ref * p.scale_log2;

            // pass 2: P = exp2(S * scale_log2 - m), packed to bf16, into TMEM
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tc::ld32(tmem + lane_base + PF_COL_S + c * 32, r);
                tc::wait_ld();
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0 = ex2(fmaf(__uint_as_float(r[i]), p.scale_log2, mneg));
                    float p1 = ex2(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, mneg));
                    if (need_mask) {
                        if (j0 + c * 32 + i > row_last) p0 = 0.f;
                        if (j0 + c * 32 + i + 1 > row_last) p1 = 0.f;
                    }
                    l_run += p0 + p1;
                    pk[i / 2] = pack_bf16(p0, p1);
                }
                tc::st16(tmem + lane_base + PF_COL_P + c * 16, pk);
            }
            tc::wait_st();
            tc::fence_before_sync();
            mbar_arrive(smem_u32(&bar_p));
        }

        // epilogue: O / l -> bf16 -> global
        if (ok && n_tiles > 0) ok = mbar_wait(smem_u32(&bar_o), 0, &s_abort);
        if (ok) {
            tc::fence_after_sync();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            __nv_bfloat16* dst = p.out + (((size_t)b * p.S + gi) * p.Hq + h) * PF_D;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t r[32];
                if (n_tiles > 0) {
                    tc::ld32(tmem + lane_base + PF_COL_O + c * 32, r);
                    tc::wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = 0;
                }
                if (gi < p.S) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint4 o4;
                        o4.x = pack_bf16(__uint_as_float(r[v * 8 + 0]) * inv, __uint_as_float(r[v * 8 + 1]) * inv);
                        o4.y = pack_bf16(__uint_as_float(r[v * 8 + 2]) * inv, __uint_as_float(r[v * 8 + 3]) * inv);
                        o4.z = pack_bf16(__uint_as_float(r[v * 8 + 4]) * inv, __uint_as_float(r[v * 8 + 5]) * inv);
                        o4.w = pack_bf16(__uint_as_float(r[v * 8 + 6]) * inv, __uint_as_float(r[v * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = o4;
                    }
                }
            }
            if (p.lse && gi < p.S)
                p.lse[((size_t)b * p.Hq + h) * p.S + gi] =
                    l_run > 0.f ? (m_ref * p.scale_log2 + log2f(l_run)) * PF_LN2 : -INFINITY;
        }
    }

    // common exit: everybody arrives here (bounded waits), then TMEM is freed
    tc::fence_before_sync();
    __syncthreads();
    if (tid == 0 && s_abort) atomicExch(p.error_word, BN_ERR_TIMEOUT);
    if (warp == 5) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem, PF_TMEM_COLS);
    }
}

}  // namespace bn

using namespace bn;

extern "C" size_t bn_attn_prefill_bf16_workspace_bytes(int B, int S, int Hq, int Hkv, int D) {
    (void)Hq;
    if (B <= 0 || S <= 0 || Hkv <= 0 || D != PF_D) return 0;
    return prefill_layout(B, S, Hkv).total;
}

extern "C" int bn_attn_prefill_bf16(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S,
                                    int Hq, int Hkv, int D, float scale, float theta, int position_offset,
                                    int causal, int flags, void* workspace, size_t workspace_bytes,
                                    bn_stream_t stream) {
    if (!q || !k || !v || !out) return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_bf16: null pointer");
    if (B < 0 || S < 0 || Hq <= 0 || Hkv <= 0)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_bf16: bad shape B=%d S=%d Hq=%d Hkv=%d", B, S, Hq, Hkv);
    if (Hq % Hkv != 0) return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_bf16: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
    if (D != PF_D) return fail(BN_ERR_UNSUPPORTED, "bn_attn_prefill_bf16: head_dim=%d (64 supported)", D);
    if (position_offset < 0) return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_bf16: position_offset=%d < 0", position_offset);
    if (flags & ~BN_PREFILL_REUSE_ROTATED_K)
        return fail(BN_ERR_UNSUPPORTED, "bn_attn_prefill_bf16: flags=0x%x not understood", flags);
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
         reinterpret_cast<uintptr_t>(out)) & 15)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_bf16: q/k/v/out must be 16-byte aligned");
    if (int rc = require_sm100()) return rc;
    if (B == 0 || S == 0) return BN_OK;
    const PrefillWsLayout L = prefill_layout(B, S, Hkv);
    if (!workspace || workspace_bytes < L.total)
        return fail(BN_ERR_WORKSPACE, "bn_attn_prefill_bf16: workspace of %zu bytes given, %zu needed", workspace_bytes,
                    L.total);
    if (reinterpret_cast<uintptr_t>(workspace) & 255)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_bf16: workspace must be 256-byte aligned");
    const long long n_qtiles = (S + PF_BM - 1) / PF_BM;
    if (n_qtiles * B * Hq > 0x7fffffffLL || B > 65535)
        return fail(BN_ERR_UNSUPPORTED, "bn_attn_prefill_bf16: problem too large for one launch");

    uint8_t* ws = static_cast<uint8_t*>(workspace);
    int* error_word = reinterpret_cast<int*>(ws);
    float2* table = reinterpret_cast<float2*>(ws + L.table);
    __nv_bfloat16* krot = reinterpret_cast<__nv_bfloat16*>(ws + L.krot);
    cudaStream_t st = as_stream(stream);

    if (!(flags & BN_PREFILL_REUSE_ROTATED_K)) {
        rope_k_kernel<<<dim3(S, B), 128, 0, st>>>(static_cast<const __nv_bfloat16*>(k), krot, table, B, S, Hkv, theta,
                                                  position_offset, error_word);
        if (int rc = launch_status("bn_attn_prefill_bf16 (rope_k)")) return rc;
    }

    // K (rotated copy) and V as 4-D tensors (D, Hkv, S, B); one box = 128 keys of one KV head
    CUtensorMap tmap_k, tmap_v;
    const uint64_t dims[4] = {(uint64_t)PF_D, (uint64_t)Hkv, (uint64_t)S, (uint64_t)B};
    const uint64_t strides[3] = {(uint64_t)PF_D * 2, (uint64_t)Hkv * PF_D * 2, (uint64_t)S * Hkv * PF_D * 2};
    const uint32_t box[4] = {PF_D, 1, PF_BN, 1};
    if (int rc = make_tensor_map(&tmap_k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, krot, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
        return rc;
    if (int rc = make_tensor_map(&tmap_v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, v, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
        return rc;

    PrefillParams p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.lse = lse;
    p.table = table;
    p.error_word = error_word;
    p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.n_rep = Hq / Hkv;
    p.n_qtiles = (int)n_qtiles;
    p.position_offset = position_offset;
    p.causal = causal;
    p.scale_log2 = scale * PF_LOG2E;

    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM_BYTES);
        if (e != cudaSuccess) return fail(BN_ERR_CUDA, "cudaFuncSetAttribute(prefill): %s", cudaGetErrorString(e));
        configured_dev = dev;
    }
    prefill_kernel<<<(unsigned)(n_qtiles * B * Hq), PF_THREADS, PF_SMEM_BYTES, st>>>(tmap_k, tmap_v, p);
    return launch_status("bn_attn_prefill_bf16");
}

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
//   2. prefill_kernel: persistent, one CTA per SM, two 128-row query tiles in
//      flight, 16 softmax warps + MMA warp + TMA warp (described at the kernel).
//      prefill_kernel_v1 (flag BN_PREFILL_SINGLE_TILE_KERNEL) is the simple
//      variant kept as a second implementation for the tests: one CTA per
//      (batch, query head, 128-row query tile), two CTAs per SM, 4 softmax
//      warps (one query row per thread), TMA warp, MMA warp; TMEM (256
//      columns): S fp32 [0,128) | O fp32 [128,192) | P bf16 [192,256).
//   Both compute S = Q K^T (128x128x64, tcgen05.mma, operands in shared memory)
//   into TMEM and O += P V (128x64x128) with P read from TMEM; softmax in base 2
//   with the scale folded into the exponent; only tiles that touch the diagonal
//   are masked, tiles above it are skipped.
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
    size_t table, kmax2, krot, total;
};

static PrefillWsLayout prefill_layout(int B, int S, int Hkv) {
    PrefillWsLayout L;
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    L.table = 256;                                               // after the header (error word)
    L.kmax2 = L.table + up((size_t)S * (PF_D / 2) * sizeof(float2));   // [B][Hkv][key tiles of 128] largest |k|^2
    L.krot = L.kmax2 + up((size_t)B * Hkv * ((S + PF_BN - 1) / PF_BN) * sizeof(float));
    L.total = L.krot + up((size_t)B * S * Hkv * PF_D * sizeof(__nv_bfloat16));
    return L;
}

void prefill_bf16_workspace_layout(int B, int S, int Hkv, size_t* table, size_t* kmax2, size_t* krot, size_t* total) {
    const PrefillWsLayout L = prefill_layout(B, S, Hkv);
    *table = L.table; *kmax2 = L.kmax2; *krot = L.krot; *total = L.total;
}

// the cos/sin table alone (for a caller that produces the rotated K itself): [S][32] of position s + position_offset
__global__ void __launch_bounds__(256)
rope_table_kernel(float2* __restrict__ table, int S, float theta, int position_offset, int* __restrict__ error_word) {
    const int idx = blockIdx.x * 256 + threadIdx.x;
    if (idx == 0) *error_word = 0;
    if (idx >= S * (PF_D / 2)) return;
    const int s = idx / (PF_D / 2), i = idx % (PF_D / 2);
    const float angle = (s + position_offset) * rope_inv_freq(i, PF_D, theta);
    table[idx] = make_float2(cosf(angle), sinf(angle));
}

// ---------------------------------------------------------------------------
// launch 1: K rotation + cos/sin table
// ---------------------------------------------------------------------------
// One block per (batch element, 128-key tile), all KV heads: the block owns the tile's norm maxima, so they are plain
// stores (no global atomics, nothing to clear first), and a cos/sin pair is computed once per position and block.
constexpr int RK_THREADS = 512;
constexpr int RK_UNROLL = 4;    // 16-byte pieces a thread has in flight

__global__ void __launch_bounds__(RK_THREADS)
rope_k_kernel(const __nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ krot, float2* __restrict__ table,
              int* __restrict__ kmax2, int B, int S, int Hkv, float theta, int position_offset,
              int* __restrict__ error_word) {
    __shared__ float2 cs[PF_BN][PF_D / 2];      // 32 KB
    __shared__ int s_kmax[64];                  // per KV head (up to 64): largest |k|^2 of the tile's keys, as float bits
    const int tile = blockIdx.x, b = blockIdx.y;
    const int s0 = tile * PF_BN, npos = min(PF_BN, S - s0);
    if (tile == 0 && b == 0 && threadIdx.x == 0) *error_word = 0;
    // 16-byte pieces (4 rotation pairs) of the tile's keys: the first loads are issued before the cos/sin work
    const int chunks_per_pos = Hkv * (PF_D / 8);
    const int n_chunks = npos * chunks_per_pos;
    const uint4* src = reinterpret_cast<const uint4*>(k + ((size_t)b * S + s0) * Hkv * PF_D);
    uint4* dst = reinterpret_cast<uint4*>(krot + ((size_t)b * S + s0) * Hkv * PF_D);
    uint4 raw[RK_UNROLL];
#pragma unroll
    for (int i = 0; i < RK_UNROLL; ++i) {
        const int e = threadIdx.x + i * RK_THREADS;
        raw[i] = e < n_chunks ? __ldg(src + e) : make_uint4(0, 0, 0, 0);
    }
    if (threadIdx.x < 64) s_kmax[threadIdx.x] = 0;
    {
        const int i = threadIdx.x % (PF_D / 2);                      // the thread's rotation pair: one frequency
        const float freq = rope_inv_freq(i, PF_D, theta);
        for (int ds = threadIdx.x / (PF_D / 2); ds < npos; ds += RK_THREADS / (PF_D / 2)) {
            const float angle = (s0 + ds + position_offset) * freq;
            const float2 v = make_float2(cosf(angle), sinf(angle));
            cs[ds][i] = v;
            if (b == 0) table[(size_t)(s0 + ds) * (PF_D / 2) + i] = v;
        }
    }
    __syncthreads();
    // Rotates one 16-byte piece (4 pairs); the squared norm of the key it belongs to is summed over the 8 threads
    // that hold the key's 8 pieces (neighbouring lanes) and the tile's maximum per KV head kept in shared memory.
    // A non-negative float orders like its bit pattern, so the maxima are integer atomics.
    auto rotate = [&](uint4 x, int e, bool valid) {
        const int ds = e / chunks_per_pos, c = e % (PF_D / 8);     // position, and which 4 pairs of the head
        uint32_t w[4] = {x.x, x.y, x.z, x.w};
        float n2 = 0.f;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const float2 v = cs[valid ? ds : 0][c * 4 + t];
            const float x0 = bf16_lo(w[t]), x1 = bf16_hi(w[t]);
            w[t] = pack_bf16(x0 * v.x - x1 * v.y, x0 * v.y + x1 * v.x);
            const float y0 = bf16_lo(w[t]), y1 = bf16_hi(w[t]);
            n2 = fmaf(y0, y0, fmaf(y1, y1, n2));
        }
        n2 += __shfl_xor_sync(0xffffffffu, n2, 1);
        n2 += __shfl_xor_sync(0xffffffffu, n2, 2);
        n2 += __shfl_xor_sync(0xffffffffu, n2, 4);
        if (valid && c == 0) {
            const int hh = (e % chunks_per_pos) / (PF_D / 8);
            // a NaN or an infinity must read as "unbounded": their bit patterns are above every finite float's
            atomicMax(&s_kmax[hh & 63], n2 == n2 ? __float_as_int(n2) : 0x7fffffff);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    };
    // whole warps take part in the shuffles, so the loops run to a multiple of the block size
    for (int e0 = 0; e0 < n_chunks; e0 += RK_UNROLL * RK_THREADS) {
        uint4 nxt[RK_UNROLL];
#pragma unroll
        for (int i = 0; i < RK_UNROLL; ++i) {                        // the next round's loads before this round's work
            const int e = e0 + RK_UNROLL * RK_THREADS + threadIdx.x + i * RK_THREADS;
            nxt[i] = e < n_chunks ? __ldg(src + e) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < RK_UNROLL; ++i) {
            const int e = e0 + threadIdx.x + i * RK_THREADS;
            const uint4 y = rotate(raw[i], e, e < n_chunks);
            if (e < n_chunks) dst[e] = y;
        }
#pragma unroll
        for (int i = 0; i < RK_UNROLL; ++i) raw[i] = nxt[i];
    }
    __syncthreads();
    // (more than 64 KV heads share slots: a head then reads the maximum over the heads of its slot, still a bound)
    for (int hh = threadIdx.x; hh < Hkv; hh += RK_THREADS)
        kmax2[((size_t)b * Hkv + hh) * ((S + PF_BN - 1) / PF_BN) + tile] = s_kmax[hh & 63];
}

// ---------------------------------------------------------------------------
// launch 2: the attention kernel
// ---------------------------------------------------------------------------
struct PrefillParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    float* lse;
    const float2* table;
    const float* kmax2;                  // [B][Hkv][n_ktiles]: largest squared norm of a rotated key in a 128-key tile
    int* error_word;
    int B, S, Hq, Hkv, n_rep, n_qtiles, n_ktiles, position_offset, causal;
    float inv_bh, inv_hq, inv_n_rep;     // reciprocals of B*Hq, Hq, n_rep for the persistent kernel's unit decode
    float scale_log2;
    float bound_scale;                   // scale_log2^2 / 60^2: |q|^2 |k|^2 times this <= 1 means every exponent stays within +-60
};

__global__ void __launch_bounds__(PF_THREADS, 2)
prefill_kernel_v1(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
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
                tc::wait_ld(r);
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
                        tc::wait_ld(r);
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
                tc::wait_ld(r);
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
                    tc::wait_ld(r);
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


// ---------------------------------------------------------------------------
// launch 2, main kernel: persistent, one CTA per SM, TWO query tiles in flight,
// THREE score buffers in tensor memory
// ---------------------------------------------------------------------------
// Work unit = (batch, query head, pair of 128-row query tiles); units are ordered
// heaviest first and dealt in snake order to the CTAs (grid = number of SMs), each
// CTA walking its units in a loop.  Eighteen warps:
//   warps 0-7   softmax of query tile 2t   (warps 0-3 keys 0..63 of a step, 4-7 keys 64..127)
//   warps 8-15  softmax of query tile 2t+1 (same split)
//   warp 16     MMA issuer                  warp 17  TMA producer
// Two threads per query row: thread = (TMEM lane = row, half of the step's 128
// keys, half of the 64 output columns).
//
// The steps (query tile u, key tile j) of a CTA form ONE sequence s = 0, 1, 2, ...
// (within a unit: j ascending, tile 0 before tile 1; units one after the other).
// Step s computes its scores into buffer s % 3, and the bf16 probabilities are
// written over the scores they came from (thread (row, half) reads 16 fp32 columns
// ahead of the 8 packed columns it overwrites), so a step owns one 128-column
// buffer from its Q K^T to the end of its P V:
//   TMEM (512 columns): S/P buffers [0,128) [128,256) [256,384) | O0 [384,448) O1 [448,512)
//   P of keys 0..63 at columns [0,32) of the buffer, keys 64..127 at [64,96).
// The MMA thread issues  Q K^T(s+3)  right after  P V(s): the tensor pipe executes
// in issue order, so the new scores cannot overtake the read of the old
// probabilities, and a softmax warp normally finds the scores of its NEXT step
// (issued a step and a half earlier) already there.  With the exponent reference
// fixed (below) the steps of a tile need nothing from each other but the order of
// their P V, so the two groups of softmax warps run back to back; the exponential
// unit (16 per clock per SM: 1024 cycles for a 128x128 step against 512 tensor
// cycles at head_dim 64) is the pipe that bounds a step.
// Both tiles read the same K/V stages (K and V of a stage behind ONE barrier), so
// each K/V tile is fetched once per 256 query rows.  Q tiles are requested by TMA a
// whole unit ahead (as soon as the unit before last has released the buffer) and
// rotated in place by the tile's own softmax warps, a row per warp instruction
// (lane = rotation pair), right after the tile's last step and before its epilogue.
// Softmax is ONE pass per step with an exponent reference that starts at 0 and
// moves only when a probability would leave [2^-64, 2^64] (bf16 and fp32 keep
// their relative precision over that range).  Whether that can happen at all is
// known before the step: |q . k| <= |q| |k|, with the largest squared norm of the
// tile's rotated query rows (taken during the rotation) and of the key tile's
// rotated keys (taken by the K rotation launch).  A step whose bound keeps every
// exponent within +-60 runs with no check and NO synchronisation between warps
// beyond the two mbarriers of its score buffer.  Only an unbounded step is checked:
// the tile's eight warps OR an "out of range" flag through a 256-thread named
// barrier; if it is raised the tile asks the MMA thread to compute the step's
// scores again (the first pass has overwritten part of them), takes the true row
// maxima, rescales O and l and redoes the step, and the rest of the unit stays on
// the checked path.
// On a tile that touches the diagonal a 16-key chunk is classified per warp: all
// keys valid for its 32 rows (no mask), none (zeros, no arithmetic), or mixed.
// Named barriers are not bounded waits; they cannot hang because a warp that
// gives up (a bounded mbarrier wait ran out, or the CTA-wide abort flag was seen)
// arrives once on every named barrier it belongs to before it leaves, and every
// warp checks the abort flag after each named barrier.
// What bounds the kernel is the softmax warps' own instruction streams (96 registers per thread, four warps per
// scheduler: dependency waits are not covered), not the exponential unit: every change that adds instructions to a
// step makes it slower, even when it takes work off that unit.
// Measured and dropped on this structure (config 2; this kernel 222 - 225 us): an eighth / a quarter / half of the
// exponentials as a cubic on the FMA pipe (246 / 262 / 279 us); the softmax scale folded into the Q rotation (no gain
// at config 2, and Q * scale rounds differently from the rotated Q that the parity oracle rounds); rotating the next
// unit's Q before a unit's last step (240 us) or after its first (238 us); the common step as straight-line code and
// the diagonal step as a rolled loop (244 us, spills); two extra warps that only rotate Q (227 us); a rolled
// 16-column loop with out-of-line helpers (260 us); the two tiles as independent streams with dynamically assigned
// score buffers (277 - 288 us).
// Optional event log for performance work (compiled out unless built with -DBN_TIMELINE): the warps of CTA 0
// append (clock64, code) pairs to the caller's lse buffer, 2048 entries per warp, INSTEAD of the log-sum-exp.
#ifdef BN_TIMELINE
#ifndef BN_TL_CTA
#define BN_TL_CTA 0
#endif
#define BN_LOG(code) do { if (blockIdx.x == BN_TL_CTA && p.lse && log_n < 2048) { long long* L_ = reinterpret_cast<long long*>(p.lse) + ((size_t)(threadIdx.x / 32) * 2048 + log_n) * 2; L_[0] = clock64(); L_[1] = (long long)(code); ++log_n; } } while (0)
#else
#define BN_LOG(code) do {} while (0)
#endif
#ifdef BN_TIMELINE_MMA
#define BN_LOG_MMA(code) BN_LOG(code)
#else
#define BN_LOG_MMA(code) do {} while (0)
#endif
#ifndef BN_MMA_LEADER
#define BN_MMA_LEADER elect_one()
#endif
// Threads per query row in a softmax group: 2 (eight warps per tile, 64 keys of a step each, 96 registers per thread)
// or 1 (four warps per tile, a whole row per thread, 165 registers: -DBN_P2_TPR=1 passes the same tests and takes
// 384 us at config 2 against 222 - 225 us; 290 us with the four 16-column chunks of a half as straight-line code, which
// lets the compiler overlap them - with two threads per row that form spills at 96 registers and is no faster).
#ifndef BN_P2_TPR
#define BN_P2_TPR 2
#endif
constexpr int P2_TPR = BN_P2_TPR;
constexpr int P2_WPT = 4 * P2_TPR;             // softmax warps per query tile
constexpr int P2_SOFT = 2 * P2_WPT;            // softmax warps; then one MMA warp and one producer warp
constexpr int P2_NH = 2 / P2_TPR;              // 64-key halves of a step that one thread handles
constexpr int P2_THREADS = 32 * (P2_SOFT + 2);
constexpr int P2_NSTAGE = 4;
constexpr int P2_NSBUF = 3;                  // score / probability buffers in tensor memory
constexpr int P2_SMEM_BYTES = 1024 + PF_TILE_BYTES * (4 + 2 * P2_NSTAGE);
constexpr uint32_t P2_TMEM_COLS = 512;
constexpr uint32_t P2_COL_O = 384;

// exp2 of 16 scores -> 8 packed bf16x2; the row sum is accumulated in two independent chains.  The arithmetic is
// plain scalar FFMA / FADD: the packed two-wide forms (fma.rn.f32x2, add.rn.f32x2) were measured slower here.
// The scale, the shift and the two sums travel as register pairs (scale2, mneg2 = the value twice; sum2): in this
// form ptxas keeps the kernel inside its 96 registers without spilling.
template <bool MASK>
__device__ __forceinline__ void softmax_chunk16(uint32_t (&r)[16], uint32_t (&pk)[8], uint64_t scale2, uint64_t mneg2,
                                                int first_key, int row_last, uint64_t& sum2) {
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
        float sc, mn, dummy;
        unpack_f32x2(scale2, sc, dummy);
        unpack_f32x2(mneg2, mn, dummy);
        float p0 = ex2(fmaf(__uint_as_float(r[i]), sc, mn));
        float p1 = ex2(fmaf(__uint_as_float(r[i + 1]), sc, mn));
        if (MASK) {
            if (first_key + i > row_last) p0 = 0.f;
            if (first_key + i + 1 > row_last) p1 = 0.f;
        }
        {
            float s0_, s1_;
            unpack_f32x2(sum2, s0_, s1_);
            sum2 = pack_f32x2(s0_ + p0, s1_ + p1);
        }
        pk[i / 2] = pack_bf16(p0, p1);
    }
}

struct UnitInfo {
    int b, h, g, qp;
    int n_t[2], n_max;
};

// k / d and k % d for 0 <= k < 2^22 without the integer-division sequence: float estimate, then a correction
__device__ __forceinline__ void fast_divmod(int k, int d, float inv_d, int& q, int& r) {
    q = __float2int_rz(__int2float_rz(k) * inv_d);
    r = k - q * d;
    if (r < 0) { --q; r += d; }
    if (r >= d) { ++q; r -= d; }
}

__device__ __forceinline__ UnitInfo unit_info(const PrefillParams& p, int k) {
    UnitInfo w;
    int qi, bh, rem;
    fast_divmod(k, p.B * p.Hq, p.inv_bh, qi, bh);
    w.qp = (p.n_qtiles + 1) / 2 - 1 - qi;      // heaviest (latest) pair of query tiles first
    fast_divmod(bh, p.Hq, p.inv_hq, w.b, w.h);   // the heads of a KV group are neighbours
    fast_divmod(w.h, p.n_rep, p.inv_n_rep, w.g, rem);
    const int n_ktiles_all = (p.S + PF_BN - 1) / PF_BN;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int i0 = (2 * w.qp + u) * PF_BM;
        if (i0 >= p.S) w.n_t[u] = 0;
        else w.n_t[u] = p.causal ? min(n_ktiles_all, (i0 + PF_BM - 1 + p.position_offset) / PF_BN + 1) : n_ktiles_all;
    }
    w.n_max = max(w.n_t[0], w.n_t[1]);
    return w;
}

// Units are sorted heaviest first and dealt to the CTAs in snake order (round r runs left to right when r is
// even, right to left when odd), which keeps the per-CTA sums within one unit of each other.  -1 = no more.
__device__ __forceinline__ int unit_of(int round, int n_units) {
    const int G = gridDim.x, c = blockIdx.x;
    const int k = round * G + ((round & 1) ? G - 1 - c : c);
    return k < n_units ? k : -1;
}

// Rare paths of the MMA thread.
// Key tiles of the two query tiles of the unit of round `it`, packed n0 | n1 << 16; -1 when the CTA has no such unit.
__device__ __forceinline__ int mma_unit_tiles(const PrefillParams& p, int n_units, int it) {
    const int k = unit_of(it, n_units);
    if (k < 0) return -1;
    const UnitInfo w = unit_info(p, k);
    return w.n_t[0] | w.n_t[1] << 16;
}

__device__ __forceinline__ bool mma_wait_operands(uint32_t bar_q, uint32_t par_q, uint32_t bar_kv, uint32_t par_kv,
                                               volatile int* abort_flag) {
    if (bar_q && !mbar_wait(bar_q, par_q, abort_flag)) return false;
    return mbar_wait(bar_kv, par_kv, abort_flag);
}

__device__ __forceinline__ bool mma_scores_again(uint32_t tS, uint32_t qd, uint32_t kd, uint32_t desc_hi, uint32_t idesc,
                                              uint32_t bar_again, uint32_t bar_redone, uint32_t par, volatile int* abort_flag) {
    tc::fence_after_sync();
#pragma unroll
    for (int kk = 0; kk < PF_D / 16; ++kk) tc::mma_ss_lohi(tS, qd + kk * 2, kd + kk * 2, desc_hi, idesc, kk > 0);
    tc::commit(bar_again);
    return mbar_wait(bar_redone, par, abort_flag);
}

// 18 warps = 5 on one scheduler: 16384 / (5 * 32) leaves 96 registers per thread
__global__ void __launch_bounds__(P2_THREADS, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const PrefillParams p, const int n_units) {
    extern __shared__ uint8_t smem_raw[];
    // Q tile barriers are indexed [buffer][tile]
    __shared__ __align__(8) uint64_t bar_qfull[2][2], bar_qrot[2][2], bar_qfree[2][2];
    __shared__ __align__(8) uint64_t bar_s[P2_NSBUF], bar_p[P2_NSBUF];      // per score buffer
    __shared__ __align__(8) uint64_t bar_o[2], bar_rs[2], bar_rp[2];        // per tile: O complete; scores again / redone
    __shared__ __align__(8) uint64_t bar_kvfull[P2_NSTAGE], bar_empty[P2_NSTAGE];   // K and V of a stage arrive on one barrier
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ int s_redo[2];
                  // per tile: how many steps have asked for their scores again
    __shared__ float s_qmax2[2][2][8];         // [Q buffer][tile][warp of the tile]: largest |q|^2 of the rows it rotated
    __shared__ float s_xchg[2][2][PF_BM];      // [tile][column half][row]: exchange between the two threads of a row

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
#ifdef BN_TIMELINE
    int log_n = 0;
#endif
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = smem0;                                        // [buffer][tile] = 4 tiles
    const uint32_t sK = smem0 + PF_TILE_BYTES * 4;                    // P2_NSTAGE tiles
    const uint32_t sV = smem0 + PF_TILE_BYTES * (4 + P2_NSTAGE);      // P2_NSTAGE tiles

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            for (int u = 0; u < 2; ++u) {
                mbar_init(smem_u32(&bar_qfull[i][u]), 1);
                mbar_init(smem_u32(&bar_qrot[i][u]), P2_WPT);
                mbar_init(smem_u32(&bar_qfree[i][u]), 1);
            }
            mbar_init(smem_u32(&bar_o[i]), 1);
            mbar_init(smem_u32(&bar_rs[i]), 1);
            mbar_init(smem_u32(&bar_rp[i]), P2_WPT);
            s_redo[i] = 0;
        }
        for (int s = 0; s < P2_NSBUF; ++s) {
            mbar_init(smem_u32(&bar_s[s]), 1);
            mbar_init(smem_u32(&bar_p[s]), P2_WPT);
        }
        for (int s = 0; s < P2_NSTAGE; ++s) {
            mbar_init(smem_u32(&bar_kvfull[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        s_abort = 0;
        fence_mbar_init();
    }
    if (warp == P2_SOFT) {
        tc::tmem_alloc(smem_u32(&s_tmem_base), P2_TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = s_tmem_base;

    if (warp == P2_SOFT + 1) {
        // ---------------------------------------------------------- TMA producer
        // K/V tiles stream through a four-stage ring.  The Q tiles of a unit are requested a whole unit ahead: as
        // soon as the unit before last has released their buffer, so that the rotation warp has the whole current
        // unit to rotate them.
        if (lane == 0) {
            prefetch_tensormap(&tmap_q);
            prefetch_tensormap(&tmap_k);
            prefetch_tensormap(&tmap_v);
            int stage = 0;
            uint32_t phase = 0;
            int q_round[2] = {0, 0};      // per tile slot: the next round whose Q tile is still to be requested
            int q_cnt[2] = {0, 0};        // ... and how many have been requested (buffer and barrier parity)
            bool ok = true;
            // requests tile slot u's Q tiles up to round `upto`; with `block` the buffer is waited for
            auto load_q = [&](int u, int upto, bool block) {
                while (ok && q_round[u] <= upto) {
                    const int k = unit_of(q_round[u], n_units);
                    if (k < 0) { q_round[u] = 0x7fffffff; return; }
                    const UnitInfo w = unit_info(p, k);
                    if ((u ? w.n_t[1] : w.n_t[0]) > 0) {
                        const int buf = q_cnt[u] & 1;
                        const uint32_t par = ((q_cnt[u] >> 1) & 1) ^ 1u;
                        const uint32_t bar = smem_u32(&bar_qfree[buf][u]);
                        if (block) { ok = mbar_wait(bar, par, &s_abort); if (!ok) return; }
                        else if (!mbar_test_wait(bar, par)) return;
                        ++q_cnt[u];
                        mbar_arrive_expect_tx(smem_u32(&bar_qfull[buf][u]), PF_TILE_BYTES);
                        tma_load_4d(sQ + (buf * 2 + u) * PF_TILE_BYTES, &tmap_q, 0, w.h, (2 * w.qp + u) * PF_BM, w.b,
                                    smem_u32(&bar_qfull[buf][u]));
                    }
                    ++q_round[u];
                }
            };
            for (int it = 0; ok; ++it) {
                const int k = unit_of(it, n_units);
                if (k < 0) break;
                const UnitInfo w = unit_info(p, k);
                load_q(0, it, true);
                load_q(1, it, true);
                for (int j = 0; ok && j < w.n_max; ++j) {
                    load_q(0, it + 1, false);
                    load_q(1, it + 1, false);
                    ok = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &s_abort);
                    if (!ok) break;
                    mbar_arrive_expect_tx(smem_u32(&bar_kvfull[stage]), 2 * PF_TILE_BYTES);
                    tma_load_4d(sK + stage * PF_TILE_BYTES, &tmap_k, 0, w.g, j * PF_BN, w.b, smem_u32(&bar_kvfull[stage]));
                    tma_load_4d(sV + stage * PF_TILE_BYTES, &tmap_v, 0, w.g, j * PF_BN, w.b, smem_u32(&bar_kvfull[stage]));
                    if (++stage == P2_NSTAGE) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == P2_SOFT) {
        // ------------------------------------------------------------ MMA issuer
        // ONE thread runs this loop, and its own instruction stream is the critical resource: it shares a scheduler
        // with four busy softmax warps.  So the steady-state path is kept short and straight: one generator (for
        // the Q K^T side) whose steps travel to the P V side through a three-entry queue of packed words; K and V
        // of a stage behind one barrier, looked at once per stage; everything rare (a new unit, a wait that does
        // not succeed at once, scores wanted again) out of line.
        if (BN_MMA_LEADER) {
            constexpr uint32_t IDESC_QK = tc::idesc_bf16(PF_BM, PF_BN, 0);
            constexpr uint32_t IDESC_PV = tc::idesc_bf16(PF_BM, PF_D, 1);
            // a shared-memory descriptor is (DESC_HI : DESC_LO + the tile's address in units of 16 bytes)
            constexpr uint32_t DESC_LO = (uint32_t)(tc::smem_desc_sw128(0) & 0xffffffffu);
            constexpr uint32_t DESC_HI = (uint32_t)(tc::smem_desc_sw128(0) >> 32);
            const uint32_t dQ = DESC_LO + (sQ >> 4), dK = DESC_LO + (sK >> 4), dV = DESC_LO + (sV >> 4);
            constexpr uint32_t TILE16 = PF_TILE_BYTES >> 4;
            const uint32_t aBarS = smem_u32(&bar_s[0]), aBarP = smem_u32(&bar_p[0]);
            const uint32_t aFull = smem_u32(&bar_kvfull[0]), aEmpty = smem_u32(&bar_empty[0]);
            const uint32_t aQrot = smem_u32(&bar_qrot[0][0]), aQfree = smem_u32(&bar_qfree[0][0]);   // [buffer][tile]

            // generator state: the step whose Q K^T is issued next
            int g_it = 0, g_n0 = 0, g_n1 = 0, g_nmax = 0, g_j = 0;   // round; key tiles of the unit's two query tiles; key tile
            uint32_t g_u = 0;                   // query tile of the pair
            uint32_t g_kt = 0;                  // ring position of the step's key tile (all earlier key tiles of the CTA)
            uint32_t g_quse0 = 0, g_quse1 = 0;  // earlier units in which tile 0 / 1 existed (-> Q buffer, barrier parity)
            bool g_valid;
            auto gen_unit = [&]() {
                const int t = mma_unit_tiles(p, n_units, g_it);
                g_valid = t >= 0;
                g_n0 = t & 0xffff;
                g_n1 = t >> 16;
                g_nmax = max(g_n0, g_n1);
                g_j = 0;
                g_u = g_n0 > 0 ? 0u : 1u;
            };
            gen_unit();
            // queue entry: bit 0 tile, 1 accumulate (j > 0), 2 last step of the tile in its unit, 3 last user of the
            // K/V stage, 4-5 stage, 6 Q buffer
            uint32_t q0 = 0, q1 = 0, q2 = 0;
            int qlen = 0;
            uint32_t bq = 0, bp = 0, par_p = 0;       // score buffers of the next Q K^T / P V; parity of bar_p[bp]
            int redo0 = 0, redo1 = 0;
            uint32_t spins = 0;
            bool ok = true;

            for (;;) {
                // ---- Q K^T, up to three steps ahead of the P V.  Only the step the P V needs next is worth blocking
                // for; for the others a missing operand (the next unit's Q still being rotated) means "look again soon".
                bool pending = false;
                while (g_valid && qlen < P2_NSBUF) {
                    const uint32_t quse = g_u ? g_quse1 : g_quse0;
                    const uint32_t qslot = (quse & 1u) * 2 + g_u;         // [buffer][tile]
                    const uint32_t stage = g_kt & (P2_NSTAGE - 1);
                    if (g_j == 0 || g_u == 0 || g_j >= g_n0) {
                        // first step of a tile in its unit: is Q rotated?  first user of a K/V stage: has it landed?
                        bool ready = true;
                        if (g_j == 0) ready = mbar_test_wait(aQrot + qslot * 8, (quse >> 1) & 1u);
                        if (ready && (g_u == 0 || g_j >= g_n0)) ready = mbar_test_wait(aFull + stage * 8, (g_kt >> 2) & 1u);
                        if (!ready) {
                            if (qlen > 0) { pending = true; break; }
                            // nothing in flight: this step is the one everybody waits for
                            ok = mma_wait_operands(g_j == 0 ? aQrot + qslot * 8 : 0u, (quse >> 1) & 1u, aFull + stage * 8,
                                                   (g_kt >> 2) & 1u, &s_abort);
                            if (!ok) break;
                        }
                    }
                    tc::fence_after_sync();
                    {
                        const uint32_t qd = dQ + qslot * TILE16, kd = dK + stage * TILE16;
#pragma unroll
                        for (int kk = 0; kk < PF_D / 16; ++kk)
                            tc::mma_ss_lohi(tmem + bq * 128, qd + kk * 2, kd + kk * 2, DESC_HI, IDESC_QK, kk > 0);
                    }
                    tc::commit(aBarS + bq * 8);
                    BN_LOG_MMA(20 | g_u << 8 | g_j << 16);
                    uint32_t e = g_u | stage << 4 | (quse & 1u) << 6;
                    if (g_j > 0) e |= 2u;
                    if (g_j == (g_u ? g_n1 : g_n0) - 1) e |= 4u;
                    if (g_u == 1 || g_j >= g_n1) e |= 8u;
                    if (qlen == 0) q0 = e; else if (qlen == 1) q1 = e; else q2 = e;
                    ++qlen;
                    bq = (bq == P2_NSBUF - 1) ? 0 : bq + 1;
                    // next step: j ascending, tile 0 before tile 1, skipping steps a tile does not have
                    if (g_u == 0 && g_j < g_n1) g_u = 1;
                    else {
                        ++g_j;
                        ++g_kt;
                        g_u = g_j < g_n0 ? 0u : 1u;
                        if (g_j >= g_nmax) {
                            g_quse0 += g_n0 > 0;
                            g_quse1 += g_n1 > 0;
                            ++g_it;
                            gen_unit();
                        }
                    }
                }
                if (!ok || qlen == 0) break;

                // ---- P of the oldest step in flight, written by the eight softmax warps of its tile
                if (!mbar_try_wait(aBarP + bp * 8, par_p)) {
                    if (!pending) {
                        ok = mbar_wait(aBarP + bp * 8, par_p, &s_abort);
                        if (!ok) break;
                    } else {
                        // a Q K^T is waiting for an operand: look again at that operand (bounded, about 2 s)
                        if (++spins > (1u << 24) || s_abort) { s_abort = 1; break; }
                        continue;
                    }
                }
                spins = 0;
                const uint32_t e = q0;
                q0 = q1; q1 = q2;
                --qlen;
                const uint32_t u = e & 1u, stage = (e >> 4) & 3u;
                // read now, tested after the address arithmetic below: the load takes its time
                const int redo_now = *reinterpret_cast<volatile int*>(&s_redo[u]);
                const uint32_t tP = tmem + bp * 128, tOu = tmem + P2_COL_O + u * 64, vd = dV + stage * TILE16;
                const uint32_t qslot = ((e >> 6) & 1u) * 2 + u;
                const int seen = u ? redo1 : redo0;
                if (redo_now != seen) {
                    // the tile wants the scores of this step again (its first pass has overwritten part of them):
                    // K(j) and Q are still in place, they are released by the commits that follow the P V
                    if (u) ++redo1; else ++redo0;
                    ok = mma_scores_again(tmem + bp * 128, dQ + qslot * TILE16, dK + stage * TILE16, DESC_HI, IDESC_QK,
                                          smem_u32(&bar_rs[u]), smem_u32(&bar_rp[u]), seen & 1, &s_abort);
                    if (!ok) break;
                }
                // O_u += P V(j)
                tc::fence_after_sync();
                tc::mma_ts_lohi(tOu, tP, vd, DESC_HI, IDESC_PV, (e >> 1) & 1u);
#pragma unroll
                for (int kk = 1; kk < PF_BN / 16; ++kk)
                    tc::mma_ts_lohi(tOu, tP + (kk & 3) * 8 + (kk >> 2) * 64, vd + kk * 128, DESC_HI, IDESC_PV, 1u);
                if (e & 4u) {
                    tc::commit(smem_u32(&bar_o[u]));          // O of this unit is complete
                    tc::commit(aQfree + qslot * 8);           // and its Q tile is done with
                }
                if (e & 8u) tc::commit(aEmpty + stage * 8);   // K(j)/V(j) may be overwritten
                BN_LOG_MMA(25 | u << 8);
                if (bp == P2_NSBUF - 1) { bp = 0; par_p ^= 1u; }
                else ++bp;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------ softmax groups (warps 0..15)
        // Eight warps per query tile: TWO threads per query row, each owning 64 of a step's 128 keys (and 32 of the
        // 64 output columns).  The two threads of a row share the exponent reference.
        const int u = warp / P2_WPT;                // which query tile of the pair
        const int hf = (warp / 4) % P2_TPR;         // which half of the keys of a step (and of the O columns); 0 when a thread has both
        const int row = (warp % 4) * 32 + lane;     // TMEM lane = query row inside the tile
        const int pair_bar = 1 + u * 4 + (warp % 4);   // named barrier of the two warps that share these 32 rows
        const int tile_bar = 9 + u;                    // named barrier of the tile's warps
        const uint32_t lane_base = ((uint32_t)((warp % 4) * 32)) << 16;
        const uint32_t tO = tmem + lane_base + P2_COL_O + u * 64 + hf * 32;
        int q_use = 0;
        int sbase = 0;                              // steps of all earlier units (both tiles)
        int redo_n = 0;
        uint32_t units_done = 0;
        bool ok = true;
        // the next unit (from round `from` on) in which this group's query tile exists; it < 0: none
        auto find_unit = [&](int from, int& it, UnitInfo& w) {
            for (it = from;; ++it) {
                const int k = unit_of(it, n_units);
                if (k < 0) { it = -1; return; }
                w = unit_info(p, k);
                if ((u ? w.n_t[1] : w.n_t[0]) > 0) return;
                sbase += w.n_t[0] + w.n_t[1];
            }
        };
        // RoPE on the TMA-loaded Q tile, in place (128-byte-swizzled, K-major).  Each of the tile's warps rotates
        // its 16 or 32 rows, a row at a time with lane = rotation pair: the row of the cos/sin table is one
        // coalesced 256-byte load and the lanes touch the 32 banks of the row's 128 bytes.  Also leaves the largest
        // squared norm of the warp's rotated rows for the bound on the scores.
        auto rotate_q = [&](const UnitInfo& w) -> bool {
            const int buf = q_use & 1;
            const uint32_t par = (q_use >> 1) & 1;
            ++q_use;
            constexpr int ROWS = PF_BM / P2_WPT;        // rows per warp: 16 or 32, sixteen at a time
            unsigned row_max = 0;
            const uint32_t chunk = (uint32_t)lane >> 2;
#pragma unroll 1
            for (int rb = 0; rb < ROWS; rb += 16) {
                const int r_first = (warp % P2_WPT) * ROWS + rb;
                const int gi_first = (2 * w.qp + u) * PF_BM + r_first;
                float2 cs[16];
#pragma unroll
                for (int r = 0; r < 16; ++r) cs[r] = __ldg(p.table + (size_t)min(gi_first + r, p.S - 1) * (PF_D / 2) + lane);
                if (rb == 0 && !mbar_wait(smem_u32(&bar_qfull[buf][u]), par, &s_abort)) return false;
                const uint32_t tile = sQ + (buf * 2 + u) * PF_TILE_BYTES + r_first * 128 + (lane & 3) * 4;
#pragma unroll
                for (int r0 = 0; r0 < 16; r0 += 8) {
                    uint32_t x[8];
#pragma unroll
                    for (int r = 0; r < 8; ++r)       // row r_first + r0 + r: its low three bits are r
                        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(x[r]) : "r"(tile + (r0 + r) * 128 + ((chunk ^ r) << 4)));
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        const float2 t2 = cs[r0 + r];
                        const float x0 = bf16_lo(x[r]), x1 = bf16_hi(x[r]);
                        const uint32_t y = pack_bf16(x0 * t2.x - x1 * t2.y, x0 * t2.y + x1 * t2.x);
                        asm volatile("st.shared.b32 [%0], %1;" ::"r"(tile + (r0 + r) * 128 + ((chunk ^ r) << 4)), "r"(y) : "memory");
                        // squared norm of the rotated row, summed over the 32 lanes in fixed point (units of 2^-10,
                        // rounded up); a lane value at the cap makes the sum reach it, which reads as "unbounded"
                        const float y0 = bf16_lo(y), y1 = bf16_hi(y);
                        const float n2 = fmaf(y0, y0, y1 * y1) * 1024.f + 1.f;
                        row_max = max(row_max, __reduce_add_sync(0xffffffffu, (unsigned)(n2 <= 1.3e8f ? n2 : 1.3e8f)));   // a NaN takes the cap
                    }
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                s_qmax2[buf][u][warp % P2_WPT] = row_max >= 130000000u ? INFINITY : (float)row_max * (1.f / 1024.f);
                mbar_arrive(smem_u32(&bar_qrot[buf][u]));
            }
            return true;
        };
        int it;
        UnitInfo w;
        find_unit(0, it, w);
        if (it >= 0) ok = rotate_q(w);
        while (ok && it >= 0) {
            const int nt = u ? w.n_t[1] : w.n_t[0];
            const int n_both = min(w.n_t[0], w.n_t[1]);     // key tiles that both query tiles of the pair have
            const int b = w.b, h = w.h;
            const int i0 = (2 * w.qp + u) * PF_BM;
            const int gi = i0 + row;

            float m_ref = 0.f;         // exponent reference, raw score units (the same in both threads of a row)
            float l_run = 0.f;         // this thread's half of the row sum
            // A step whose scores are bounded needs no check at all: |q . k| <= |q| |k|, with the largest |q|^2 of
            // the tile's rotated rows (left by the rotation) and the largest |k|^2 of the key tile (left by the K
            // rotation launch).  q_bound * |k|^2 <= 1 means that every exponent of the step lies within +-60.
            float q_bound = 0.f;       // set at the unit's first step
            bool moved = false;        // the reference has left 0 in this unit: every later step is checked
            const float* kmax2 = p.kmax2 + ((size_t)b * p.Hkv + w.g) * p.n_ktiles;
            const int row_last = p.causal ? min(p.S - 1, gi + p.position_offset) : p.S - 1;
            const int tile_free_last = p.causal ? min(p.S - 1, i0 + p.position_offset) : p.S - 1;   // no mask needed up to here
            // last valid key of the first and of the last row of this warp's 32 rows
            const int warp_first_last = p.causal ? min(p.S - 1, gi - lane + p.position_offset) : p.S - 1;
            const int warp_last_last = p.causal ? min(p.S - 1, gi - lane + 31 + p.position_offset) : p.S - 1;

            for (int j = 0; j < nt; ++j) {
                // this step's place in the CTA's sequence, hence its score buffer
                const uint32_t s = (uint32_t)(sbase + (j < n_both ? 2 * j + u : n_both + j));
                const uint32_t sb = s % P2_NSBUF;
                const uint32_t tS = tmem + lane_base + sb * 128 + hf * 64;   // 64 fp32 scores; P goes over the first 32
                BN_LOG(1 | u << 8 | j << 16);
                const float k_max2 = __ldg(kmax2 + j);
                ok = mbar_wait(smem_u32(&bar_s[sb]), (s / P2_NSBUF) & 1, &s_abort);
                if (!ok) break;
                tc::fence_after_sync();
                BN_LOG(2 | u << 8 | j << 16);
                if (j == 0) {
                    // written by the tile's eight warps before they arrived on the barrier the MMA thread waited
                    // for before this step's Q K^T
                    const volatile float* qm = s_qmax2[(q_use - 1) & 1][u];
                    float m2 = qm[0];
#pragma unroll
                    for (int i = 1; i < P2_WPT; ++i) m2 = fmaxf(m2, qm[i]);
                    q_bound = m2 * p.bound_scale;
                }
                const bool bounded = !moved && (q_bound * k_max2 <= 1.0f);
                const int j0 = j * PF_BN + hf * 64;             // first key of this thread's 64 columns
                const bool need_mask = (j0 + 64 * P2_NH - 1) > tile_free_last;    // some key of the thread's columns is masked for some row of the tile

                // One pass over this thread's 64 columns: P = exp2(S * scale_log2 - m_ref * scale_log2), each 8 packed
                // columns written over scores that have already been read.  A 16-column chunk is decided for the
                // warp: all 16 keys valid for its 32 rows -> no mask; none of them -> zeros without any arithmetic;
                // else the masked form.
                // The exponent reference starts at 0 and moves only when it has to: p = 2^(s*c - ref) may be
                // anywhere in [2^-64, 2^64] without any loss (bf16 and fp32 keep their relative precision over
                // that range), so for ordinary score magnitudes there is never a second pass or an O rescale.
                float lsum;
                bool second = false;
                for (;;) {
                    {
                        uint64_t sum2 = 0;   // (0.f, 0.f)
                        const float mneg = -m_ref * p.scale_log2;
                        const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2), mneg2 = pack_f32x2(mneg, mneg);
                        uint32_t r0[16], r1[16], pk[8];
#pragma unroll
                        for (int hh = 0; hh < P2_NH; ++hh) {       // the thread's 64-key halves of the step: one or two
                            const uint32_t tSh = tS + hh * 64;
                            const int j0h = j0 + hh * 64;
                            const bool need_mask_h = (j0h + 63) > tile_free_last;
                            auto chunk = [&](uint32_t (&r)[16], int c) {
                                const int kc = j0h + c * 16;
                                if (!need_mask_h || kc + 15 <= warp_first_last) softmax_chunk16<false>(r, pk, scale2, mneg2, kc, row_last, sum2);
                                else if (kc > warp_last_last) {
#pragma unroll
                                    for (int i = 0; i < 8; ++i) pk[i] = 0u;
                                } else softmax_chunk16<true>(r, pk, scale2, mneg2, kc, row_last, sum2);
                            };
                            // the load of the next 16 columns is in flight while the current 16 are processed
                            tc::ld16(tSh + 0, r0);
                            tc::wait_ld(r0);
                            tc::ld16(tSh + 16, r1);
                            chunk(r0, 0);
                            tc::st8(tSh + 0, pk);
                            tc::wait_ld(r1);
                            tc::ld16(tSh + 32, r0);
                            chunk(r1, 1);
                            tc::st8(tSh + 8, pk);
                            tc::wait_ld(r0);
                            tc::ld16(tSh + 48, r1);
                            chunk(r0, 2);
                            tc::st8(tSh + 16, pk);
                            tc::wait_ld(r1);
                            chunk(r1, 3);
                            tc::st8(tSh + 24, pk);
                        }
                        float s0, s1;
                        unpack_f32x2(sum2, s0, s1);
                        lsum = s0 + s1;
                    }
                    if (bounded || second) break;
                    const bool over = !(lsum <= 0x1p64f) || (j == 0 && hf == 0 && lsum < 0x1p-64f);
                    const bool redo = named_bar_or(tile_bar, 32 * P2_WPT, over);
                    if (s_abort) { ok = false; break; }
                    if (!redo) break;
                    // Rare, and taken by the whole tile together.  The first pass has overwritten scores, so the
                    // MMA thread computes them again; its commit also tells that every earlier P V of this tile has
                    // completed, so O may be rescaled here.
                    moved = true;
                    second = true;
                    tc::wait_st();
                    tc::fence_before_sync();
                    ++redo_n;
                    if ((warp % P2_WPT) == 0 && lane == 0) *reinterpret_cast<volatile int*>(&s_redo[u]) = redo_n;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bar_p[sb]));
                    ok = mbar_wait(smem_u32(&bar_rs[u]), (redo_n - 1) & 1, &s_abort);
                    if (!ok) break;
                    tc::fence_after_sync();
                    float hmax = -INFINITY;
#pragma unroll 1
                    for (int c = 0; c < 4 * P2_NH; ++c) {
                        uint32_t r[16];
                        const int col = (c >> 2) * 64 + (c & 3) * 16;
                        tc::ld16(tS + col, r);
                        tc::wait_ld(r);
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (!need_mask || j0 + col + i <= row_last) hmax = fmaxf(hmax, __uint_as_float(r[i]));
                    }
                    float tmax = hmax;
                    if (P2_TPR == 2) {
                        s_xchg[u][hf][row] = hmax;
                        named_bar_sync(pair_bar, 64);
                        if (s_abort) { ok = false; break; }
                        tmax = fmaxf(hmax, s_xchg[u][hf ^ 1][row]);
                    }
                    const float m_new = j == 0 ? tmax : fmaxf(m_ref, tmax);   // the first step may also move it down
                    const float m_upd = m_new == -INFINITY ? m_ref : m_new;
                    if (j > 0) {
                        const float alpha = ex2((m_ref - m_upd) * p.scale_log2);
                        l_run *= alpha;
#pragma unroll 1
                        for (int c = 0; c < 2 * P2_NH; ++c) {       // this thread's 32 (or all 64) O columns
                            uint32_t ro[16];
                            tc::ld16(tO + c * 16, ro);
                            tc::wait_ld(ro);
#pragma unroll
                            for (int i = 0; i < 16; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * alpha);
                            tc::st16(tO + c * 16, ro);
                        }
                    }
                    m_ref = m_upd;
                }
                if (!ok) break;
                if (second && P2_TPR == 2) {
                    named_bar_sync(pair_bar, 64);      // the exchange slots may be written again
                    if (s_abort) { ok = false; break; }
                }
                l_run += lsum;
                tc::wait_st();
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(second ? smem_u32(&bar_rp[u]) : smem_u32(&bar_p[sb]));
                BN_LOG(6 | u << 8 | j << 16);
            }
            if (!ok) break;
            sbase += w.n_t[0] + w.n_t[1];

            // The next unit's Q tile is rotated BEFORE this unit's epilogue: the MMA thread needs it to start the
            // next unit, while the epilogue has to wait for the last P V anyway.
            int it_next;
            UnitInfo w_next;
            find_unit(it + 1, it_next, w_next);
            if (it_next >= 0) {
                ok = rotate_q(w_next);
                if (!ok) break;
            }


            // epilogue: O / l -> bf16 -> global; each thread of a row writes its 32 columns
            ok = mbar_wait(smem_u32(&bar_o[u]), units_done & 1, &s_abort);
            ++units_done;
            if (!ok) break;
            tc::fence_after_sync();
            float l_row = l_run;
            if (P2_TPR == 2) {
                s_xchg[u][hf][row] = l_run;
                named_bar_sync(pair_bar, 64);
                l_row = l_run + s_xchg[u][hf ^ 1][row];
            }
            const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
            __nv_bfloat16* dst = p.out + (((size_t)b * p.S + gi) * p.Hq + h) * PF_D + hf * 32;
            // the next unit's first P V overwrites O only after this group's next P arrive, which follows these loads
#pragma unroll 1
            for (int oh = 0; oh < P2_NH; ++oh) {
                uint32_t ro[32];
                tc::ld32(tO + oh * 32, ro);
                tc::wait_ld(ro);
                if (gi < p.S) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint4 o4;
                        o4.x = pack_bf16(__uint_as_float(ro[v * 8 + 0]) * inv, __uint_as_float(ro[v * 8 + 1]) * inv);
                        o4.y = pack_bf16(__uint_as_float(ro[v * 8 + 2]) * inv, __uint_as_float(ro[v * 8 + 3]) * inv);
                        o4.z = pack_bf16(__uint_as_float(ro[v * 8 + 4]) * inv, __uint_as_float(ro[v * 8 + 5]) * inv);
                        o4.w = pack_bf16(__uint_as_float(ro[v * 8 + 6]) * inv, __uint_as_float(ro[v * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + oh * 32 + v * 8) = o4;
                    }
                }
            }
#ifndef BN_TIMELINE
            if (gi < p.S && p.lse && hf == 0)
                p.lse[((size_t)b * p.Hq + h) * p.S + gi] =
                    l_row > 0.f ? (m_ref * p.scale_log2 + log2f(l_row)) * PF_LN2 : -INFINITY;
#endif
            // the partner reads this thread's exchange slot before either of them can write it again: the next
            // write is behind the tile barrier of the next step, or behind the partner's own arrival at the next
            // epilogue's pair barrier
            it = it_next;
            w = w_next;
        }
        // a warp that gives up (a bounded wait ran out) releases whoever may be waiting for it at a named barrier
        if (!ok) {
            if (P2_TPR == 2) named_bar_arrive(pair_bar, 64);
            named_bar_arrive(tile_bar, 32 * P2_WPT);
        }
    }

    // common exit: everybody arrives here (all waits are bounded), then TMEM is freed
    tc::fence_before_sync();
    __syncthreads();
    if (tid == 0 && s_abort) atomicExch(p.error_word, BN_ERR_TIMEOUT);
    if (warp == P2_SOFT) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem, P2_TMEM_COLS);
    }
}

}  // namespace bn

using namespace bn;

extern "C" size_t bn_attn_prefill_bf16_workspace_bytes(int B, int S, int Hq, int Hkv, int D) {
    (void)Hq;
    if (B <= 0 || S <= 0 || Hkv <= 0 || D != PF_D) return 0;
    return prefill_layout(B, S, Hkv).total;
}

extern "C" int bn_attn_prefill_bf16_table(int B, int S, int Hkv, int D, float theta, int position_offset, void* workspace,
                                          size_t workspace_bytes, bn_stream_t stream) {
    if (B <= 0 || S <= 0 || Hkv <= 0 || position_offset < 0)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_bf16_table: bad shape B=%d S=%d Hkv=%d", B, S, Hkv);
    if (D != PF_D) return fail(BN_ERR_UNSUPPORTED, "bn_attn_prefill_bf16_table: head_dim=%d (64 supported)", D);
    const PrefillWsLayout L = prefill_layout(B, S, Hkv);
    if (!workspace || workspace_bytes < L.total)
        return fail(BN_ERR_WORKSPACE, "bn_attn_prefill_bf16_table: workspace of %zu bytes given, %zu needed", workspace_bytes,
                    L.total);
    if (reinterpret_cast<uintptr_t>(workspace) & 255)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_bf16_table: workspace must be 256-byte aligned");
    if (int rc = require_sm100()) return rc;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    rope_table_kernel<<<(S * (PF_D / 2) + 255) / 256, 256, 0, as_stream(stream)>>>(
        reinterpret_cast<float2*>(ws + L.table), S, theta, position_offset, reinterpret_cast<int*>(ws));
    return launch_status("bn_attn_prefill_bf16_table");
}

extern "C" int bn_attn_prefill_bf16(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S,
                                    int Hq, int Hkv, int D, float scale, float theta, int position_offset,
                                    int causal, int flags, void* workspace, size_t workspace_bytes,
                                    bn_stream_t stream) {
    if (!q || !v || !out || (!k && !(flags & BN_PREFILL_REUSE_ROTATED_K)))
        return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_bf16: null pointer");
    if (B < 0 || S < 0 || Hq <= 0 || Hkv <= 0)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_bf16: bad shape B=%d S=%d Hq=%d Hkv=%d", B, S, Hq, Hkv);
    if (Hq % Hkv != 0) return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_bf16: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
    if (D != PF_D) return fail(BN_ERR_UNSUPPORTED, "bn_attn_prefill_bf16: head_dim=%d (64 supported)", D);
    if (position_offset < 0) return fail(BN_ERR_INVALID_ARG, "bn_attn_prefill_bf16: position_offset=%d < 0", position_offset);
    if (flags & ~(BN_PREFILL_REUSE_ROTATED_K | BN_PREFILL_SINGLE_TILE_KERNEL))
        return fail(BN_ERR_UNSUPPORTED, "bn_attn_prefill_bf16: flags=0x%x not understood", flags);
    if ((reinterpret_cast<uintptr_t>(q) | (k ? reinterpret_cast<uintptr_t>(k) : 0) | reinterpret_cast<uintptr_t>(v) |
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

    int* kmax2 = reinterpret_cast<int*>(ws + L.kmax2);
    if (!(flags & BN_PREFILL_REUSE_ROTATED_K)) {
        rope_k_kernel<<<dim3((S + PF_BN - 1) / PF_BN, B), RK_THREADS, 0, st>>>(static_cast<const __nv_bfloat16*>(k), krot, table,
                                                                          kmax2, B, S, Hkv, theta, position_offset, error_word);
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
    // Q as (D, Hq, S, B); one box = 128 query rows of one head
    CUtensorMap tmap_q;
    const uint64_t qdims[4] = {(uint64_t)PF_D, (uint64_t)Hq, (uint64_t)S, (uint64_t)B};
    const uint64_t qstrides[3] = {(uint64_t)PF_D * 2, (uint64_t)Hq * PF_D * 2, (uint64_t)S * Hq * PF_D * 2};
    if (int rc = make_tensor_map(&tmap_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, q, qdims, qstrides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
        return rc;

    PrefillParams p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.lse = lse;
    p.table = table;
    p.kmax2 = reinterpret_cast<const float*>(kmax2);
    p.n_ktiles = (S + PF_BN - 1) / PF_BN;
    p.error_word = error_word;
    p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.n_rep = Hq / Hkv;
    p.n_qtiles = (int)n_qtiles;
    p.position_offset = position_offset;
    p.causal = causal;
    p.scale_log2 = scale * PF_LOG2E;
    p.bound_scale = p.scale_log2 * p.scale_log2 / 3600.f;

    static thread_local int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P2_SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(prefill_kernel_v1, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM_BYTES);
        if (e != cudaSuccess) return fail(BN_ERR_CUDA, "cudaFuncSetAttribute(prefill): %s", cudaGetErrorString(e));
        configured_dev = dev;
    }
    if (flags & BN_PREFILL_SINGLE_TILE_KERNEL) {
        prefill_kernel_v1<<<(unsigned)(n_qtiles * B * Hq), PF_THREADS, PF_SMEM_BYTES, st>>>(tmap_k, tmap_v, p);
    } else {
        const long long n_units = (long long)(n_qtiles + 1) / 2 * B * Hq;
        if (n_units >= (1ll << 22)) return fail(BN_ERR_UNSUPPORTED, "bn_attn_prefill_bf16: more than 2^22 work units");
        p.inv_bh = 1.0f / (float)(B * Hq);
        p.inv_hq = 1.0f / (float)Hq;
        p.inv_n_rep = 1.0f / (float)p.n_rep;
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const unsigned grid = (unsigned)(n_units < sms ? n_units : sms);
        prefill_kernel<<<grid, P2_THREADS, P2_SMEM_BYTES, st>>>(tmap_q, tmap_k, tmap_v, p, (int)n_units);
    }
    return launch_status("bn_attn_prefill_bf16");
}

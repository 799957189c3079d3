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
constexpr int RK_POS = 8;   // positions per block

__global__ void __launch_bounds__(256)
rope_k_kernel(const __nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ krot, float2* __restrict__ table, int B,
              int S, int Hkv, float theta, int position_offset, int* __restrict__ error_word) {
    __shared__ float2 cs[RK_POS][PF_D / 2];
    const int s0 = blockIdx.x * RK_POS, b = blockIdx.y;
    if (blockIdx.x == 0 && b == 0 && threadIdx.x == 0) *error_word = 0;
    // 16-byte pieces (4 rotation pairs) of this block's positions: issue the loads before the cos/sin work
    const int chunks_per_pos = Hkv * (PF_D / 8);
    const int n_chunks = min(RK_POS, S - s0) * chunks_per_pos;
    const uint4* src = reinterpret_cast<const uint4*>(k + ((size_t)b * S + s0) * Hkv * PF_D);
    uint4* dst = reinterpret_cast<uint4*>(krot + ((size_t)b * S + s0) * Hkv * PF_D);
    constexpr int RK_UNROLL = 2;
    uint4 raw[RK_UNROLL];
#pragma unroll
    for (int i = 0; i < RK_UNROLL; ++i) {
        const int e = threadIdx.x + i * 256;
        raw[i] = e < n_chunks ? __ldg(src + e) : make_uint4(0, 0, 0, 0);
    }
    {
        const int ds = threadIdx.x / (PF_D / 2), i = threadIdx.x % (PF_D / 2);
        const float freq = rope_inv_freq(i, PF_D, theta);
        const float angle = (s0 + ds + position_offset) * freq;
        const float2 v = make_float2(cosf(angle), sinf(angle));
        cs[ds][i] = v;
        if (b == 0 && s0 + ds < S) table[(size_t)(s0 + ds) * (PF_D / 2) + i] = v;
    }
    __syncthreads();
    auto rotate = [&](uint4 x, int e) {
        const int ds = e / chunks_per_pos, c = e % (PF_D / 8);     // position, and which 4 pairs of the head
        uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const float2 v = cs[ds][c * 4 + t];
            const float x0 = bf16_lo(w[t]), x1 = bf16_hi(w[t]);
            w[t] = pack_bf16(x0 * v.x - x1 * v.y, x0 * v.y + x1 * v.x);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    };
#pragma unroll
    for (int i = 0; i < RK_UNROLL; ++i) {
        const int e = threadIdx.x + i * 256;
        if (e < n_chunks) dst[e] = rotate(raw[i], e);
    }
    for (int e = threadIdx.x + RK_UNROLL * 256; e < n_chunks; e += 256) dst[e] = rotate(__ldg(src + e), e);
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
    float inv_bh, inv_hq, inv_n_rep;     // reciprocals of B*Hq, Hq, n_rep for the persistent kernel's unit decode
    float scale_log2;
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
// launch 2, main kernel: persistent, one CTA per SM, TWO query tiles in flight
// ---------------------------------------------------------------------------
// Work unit = (batch, query head, pair of 128-row query tiles); units are ordered
// heaviest first and dealt in snake order to the CTAs (grid = number of SMs), each
// CTA walking its units in a loop so that the next unit's Q/K/V loads overlap the
// current unit's tail.  Eighteen warps:
//   warps 0-7   softmax of query tile 2t   (warps 0-3 keys 0..63 of a step, 4-7 keys 64..127)
//   warps 8-15  softmax of query tile 2t+1 (same split)
//   warp 16     MMA issuer                  warp 17  TMA producer
// Two threads per query row: thread = (TMEM lane = row, half of the step's 128
// keys, half of the 64 output columns).  Four softmax warps per scheduler hide
// the latencies of TMEM loads, barrier waits and exponentials; the two threads
// of a row share the exponent reference, their per-step exchange is one named
// barrier (64 threads) that ORs an "out of range" flag.
// Both tiles read the same K/V stages, so each K/V tile is fetched once per
// 256 query rows, and the tensor pipe works on one tile (next Q K^T, then P V)
// while the other tile's softmax runs.  Q tiles arrive by TMA (double buffered
// across units) and are rotated in place, a row per warp instruction (lane =
// rotation pair), one unit AHEAD: right after a tile's last step and before its
// epilogue, so the MMA warp can start the next unit while O is written out.
// TMEM (512 columns): S0 [0,128) S1 [128,256) O0 [256,320) O1 [320,384)
//                     P0 [384,448) P1 [448,512)
// Softmax is ONE pass per step with an exponent reference that starts at 0 and
// moves only when a probability would leave [2^-64, 2^64] (bf16 and fp32 keep
// their relative precision over that range): then the two warps of the rows
// take the true row maximum, rescale O and l and redo the step.
// What bounds it (measured): with the exponential replaced by an FMA the kernel
// still takes 87 % of its time, so the chain  S ready -> TMEM loads -> P stored ->
// MMA warp wakes -> next Q K^T issued, executed, committed  (about 850 cycles of
// it pure hand-off latency per step and tile), not MUFU or the tensor pipe, is
// the limit; TMEM has no room for a second S buffer per tile at 128-key steps.
// Measured and dropped: exponentials on the FMA pipe; 64-key steps with double-
// buffered S; one MMA warp per tile; pairing two heads on the same query rows;
// an extra warp for the Q rotation; issuing P V before the next Q K^T.
// Optional event log for performance work (compiled out unless built with -DBN_TIMELINE): the warps of CTA 0
// append (clock64, code) pairs to the caller's lse buffer, 2048 entries per warp, INSTEAD of the log-sum-exp.
#ifdef BN_TIMELINE
#define BN_LOG(code) do { if (blockIdx.x == 0 && p.lse && log_n < 2048) { long long* L_ = reinterpret_cast<long long*>(p.lse) + ((size_t)(threadIdx.x / 32) * 2048 + log_n) * 2; L_[0] = clock64(); L_[1] = (long long)(code); ++log_n; } } while (0)
#else
#define BN_LOG(code) do {} while (0)
#endif
constexpr int P2_THREADS = 576;
constexpr int P2_NSTAGE = 4;
constexpr int P2_SMEM_BYTES = 1024 + PF_TILE_BYTES * (4 + 2 * P2_NSTAGE);
constexpr uint32_t P2_TMEM_COLS = 512;

// exp2 of 16 scores -> 8 packed bf16x2; the row sum is accumulated in two independent chains.  The arithmetic is
// plain scalar FFMA / FADD: the packed two-wide forms (fma.rn.f32x2, add.rn.f32x2) were measured slower here.
// The scale, the shift and the two sums travel as register pairs (scale2, mneg2 = the value twice; sum2): in this
// form ptxas keeps the kernel inside its 96 registers without spilling, which is worth 4 % of the run time.
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

// 18 warps = 5 on one scheduler: 16384 / (5 * 32) leaves 96 registers per thread
__global__ void __launch_bounds__(P2_THREADS, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const PrefillParams p, const int n_units) {
    extern __shared__ uint8_t smem_raw[];
    // Q tile barriers are indexed [buffer][tile]
    __shared__ __align__(8) uint64_t bar_qfull[2][2], bar_qrot[2][2], bar_qfree[2][2];
    __shared__ __align__(8) uint64_t bar_s[2], bar_p[2], bar_o[2], bar_pv[2];
    __shared__ __align__(8) uint64_t bar_kfull[P2_NSTAGE], bar_vfull[P2_NSTAGE], bar_empty[P2_NSTAGE];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
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
                mbar_init(smem_u32(&bar_qrot[i][u]), 8);
                mbar_init(smem_u32(&bar_qfree[i][u]), 1);
            }
            mbar_init(smem_u32(&bar_s[i]), 1);
            mbar_init(smem_u32(&bar_p[i]), 8);
            mbar_init(smem_u32(&bar_o[i]), 1);
            mbar_init(smem_u32(&bar_pv[i]), 1);
        }
        for (int s = 0; s < P2_NSTAGE; ++s) {
            mbar_init(smem_u32(&bar_kfull[s]), 1);
            mbar_init(smem_u32(&bar_vfull[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        s_abort = 0;
        fence_mbar_init();
    }
    if (warp == 16) {
        tc::tmem_alloc(smem_u32(&s_tmem_base), P2_TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = s_tmem_base;

    if (warp == 17) {
        // ---------------------------------------------------------- TMA producer
        if (lane == 0) {
            prefetch_tensormap(&tmap_q);
            prefetch_tensormap(&tmap_k);
            prefetch_tensormap(&tmap_v);
            int stage = 0;
            uint32_t phase = 0;
            int q_use[2] = {0, 0};        // how many units have used tile slot u so far
            bool ok = true;
            for (int it = 0; ok; ++it) {
                const int k = unit_of(it, n_units);
                if (k < 0) break;
                const UnitInfo w = unit_info(p, k);
                for (int u = 0; u < 2 && ok; ++u) {
                    if (w.n_t[u] == 0) continue;
                    const int buf = q_use[u] & 1;
                    const uint32_t par = (q_use[u] >> 1) & 1;
                    ++q_use[u];
                    ok = mbar_wait(smem_u32(&bar_qfree[buf][u]), par ^ 1u, &s_abort);
                    if (!ok) break;
                    mbar_arrive_expect_tx(smem_u32(&bar_qfull[buf][u]), PF_TILE_BYTES);
                    tma_load_4d(sQ + (buf * 2 + u) * PF_TILE_BYTES, &tmap_q, 0, w.h, (2 * w.qp + u) * PF_BM, w.b,
                                smem_u32(&bar_qfull[buf][u]));
                }
                for (int j = 0; ok && j < w.n_max; ++j) {
                    ok = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &s_abort);
                    if (!ok) break;
                    mbar_arrive_expect_tx(smem_u32(&bar_kfull[stage]), PF_TILE_BYTES);
                    tma_load_4d(sK + stage * PF_TILE_BYTES, &tmap_k, 0, w.g, j * PF_BN, w.b, smem_u32(&bar_kfull[stage]));
                    mbar_arrive_expect_tx(smem_u32(&bar_vfull[stage]), PF_TILE_BYTES);
                    tma_load_4d(sV + stage * PF_TILE_BYTES, &tmap_v, 0, w.g, j * PF_BN, w.b, smem_u32(&bar_vfull[stage]));
                    if (++stage == P2_NSTAGE) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 16) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t IDESC_QK = tc::idesc_bf16(PF_BM, PF_BN, 0);
        constexpr uint32_t IDESC_PV = tc::idesc_bf16(PF_BM, PF_D, 1);
        // a shared-memory descriptor is this constant plus the tile's address in units of 16 bytes (bits 0-13)
        const uint64_t dZero = tc::smem_desc_sw128(0);
        int stage = 0;
        uint32_t phase = 0;
        int q_use[2] = {0, 0};
        uint32_t tiles_done[2] = {0, 0};    // tiles of slot u completed so far (parity of bar_s / bar_p)
        uint32_t units_done[2] = {0, 0};
        bool ok = true;
        for (int it = 0; ok; ++it) {
            const int k = unit_of(it, n_units);
            if (k < 0) break;
            const UnitInfo w = unit_info(p, k);
            uint32_t qaddr[2] = {0, 0};
            for (int u = 0; u < 2 && ok; ++u) {
                if (w.n_t[u] == 0) continue;
                const int buf = q_use[u] & 1;
                const uint32_t par = (q_use[u] >> 1) & 1;
                ++q_use[u];
                qaddr[u] = sQ + (buf * 2 + u) * PF_TILE_BYTES;
                ok = mbar_wait(smem_u32(&bar_qrot[buf][u]), par, &s_abort);
            }
            if (!ok) break;
            // S_u = Q_u K(j)^T; the last one of the unit also frees the Q buffer
            auto issue_qk = [&](int u, int st, int j) {
                if (elect_one()) {
                    tc::fence_after_sync();
#pragma unroll
                    for (int kk = 0; kk < PF_D / 16; ++kk)
                        tc::mma_ss(tmem + u * 128, dZero + (uint64_t)((qaddr[u] >> 4) + kk * 2),
                                   dZero + (uint64_t)(((sK + st * PF_TILE_BYTES) >> 4) + kk * 2), IDESC_QK, kk > 0);
                    tc::commit(smem_u32(&bar_s[u]));
                    if (j == w.n_t[u] - 1) tc::commit(smem_u32(&bar_qfree[(q_use[u] - 1) & 1][u]));
                }
                __syncwarp();
            };
            if (w.n_max > 0) ok = mbar_wait(smem_u32(&bar_kfull[stage]), phase, &s_abort);
            if (!ok) break;
            if (elect_one()) BN_LOG(20);
            if (w.n_t[0] > 0) issue_qk(0, stage, 0);
            if (w.n_t[1] > 0) issue_qk(1, stage, 0);
            if (elect_one()) BN_LOG(21);
            for (int j = 0; ok && j < w.n_max; ++j) {
                const int nstage = (stage + 1 == P2_NSTAGE) ? 0 : stage + 1;
                const uint32_t nphase = (stage + 1 == P2_NSTAGE) ? phase ^ 1u : phase;
                bool next_k_ready = false;
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    if (j >= w.n_t[u]) continue;
                    ok = mbar_wait(smem_u32(&bar_p[u]), (tiles_done[u] + j) & 1, &s_abort);
                    if (!ok) break;
                    if (elect_one()) BN_LOG(24 | u << 8 | j << 16);
                    // S_u(j+1) = Q_u K(j+1)^T first: its S columns are free because P_u(j) has been written, and
                    // the softmax of tile j+1 can start while P_u(j) V(j) still runs
                    if (j + 1 < w.n_t[u]) {
                        if (!next_k_ready) {
                            ok = mbar_wait(smem_u32(&bar_kfull[nstage]), nphase, &s_abort);
                            if (!ok) break;
                            next_k_ready = true;
                        }
                        issue_qk(u, nstage, j + 1);
                    }
                    // O_u += P_u(j) V(j)
                    ok = mbar_wait(smem_u32(&bar_vfull[stage]), phase, &s_abort);
                    if (!ok) break;
                    if (elect_one()) {
                        tc::fence_after_sync();
#pragma unroll
                        for (int kk = 0; kk < PF_BN / 16; ++kk)
                            tc::mma_ts(tmem + 256 + u * 64, tmem + 384 + u * 64 + kk * 8,
                                       dZero + (uint64_t)(((sV + stage * PF_TILE_BYTES) >> 4) + kk * 128), IDESC_PV,
                                       (j > 0) || (kk > 0));
                        tc::commit(smem_u32(&bar_pv[u]));                          // P_u(j) may be overwritten
                        if (j == w.n_t[u] - 1) tc::commit(smem_u32(&bar_o[u]));
                        const bool last_user = (u == 1) || (j >= w.n_t[1]);
                        if (last_user) tc::commit(smem_u32(&bar_empty[stage]));   // K(j)/V(j) may be overwritten
                        BN_LOG(25 | u << 8 | j << 16);
                    }
                    __syncwarp();
                }
                stage = nstage;
                phase = nphase;
            }
            tiles_done[0] += w.n_t[0];
            tiles_done[1] += w.n_t[1];
            units_done[0] += w.n_t[0] > 0;
            units_done[1] += w.n_t[1] > 0;
        }
    } else {
        // ------------------------------------------ softmax groups (warps 0..15)
        // Eight warps per query tile: TWO threads per query row, each owning 64 of a step's 128 keys (and 32 of the
        // 64 output columns).  Four softmax warps per scheduler instead of two hide the latencies of TMEM loads,
        // barrier waits and the exponential's result.  The two threads of a row share the exponent reference;
        // their only per-step exchange is one named barrier that ORs the "probability left the safe range" flag.
        const int u = warp / 8;                     // which query tile of the pair
        const int hf = (warp / 4) % 2;              // which half of the keys of a step (and of the O columns)
        const int row = (warp % 4) * 32 + lane;     // TMEM lane = query row inside the tile
        const int pair_bar = 1 + u * 4 + (warp % 4);   // named barrier of the two warps that share these 32 rows
        const uint32_t lane_base = ((uint32_t)((warp % 4) * 32)) << 16;
        const uint32_t tS = tmem + lane_base + u * 128 + hf * 64;
        const uint32_t tO = tmem + lane_base + 256 + u * 64 + hf * 32;
        const uint32_t tP = tmem + lane_base + 384 + u * 64 + hf * 32;
        int q_use = 0;
        uint32_t tiles_done = 0, units_done = 0;
        bool ok = true;
        // the next unit (from round `from` on) in which this group's query tile exists; it < 0: none
        auto find_unit = [&](int from, int& it, UnitInfo& w) {
            for (it = from;; ++it) {
                const int k = unit_of(it, n_units);
                if (k < 0) { it = -1; return; }
                w = unit_info(p, k);
                if (w.n_t[u] > 0) return;
            }
        };
        // RoPE on the TMA-loaded Q tile, in place (128-byte-swizzled, K-major).  Each of the tile's eight warps
        // rotates 16 rows, a row at a time with lane = rotation pair: the row of the cos/sin table is one
        // coalesced 256-byte load and the lanes touch the 32 banks of the row's 128 bytes.
        auto rotate_q = [&](const UnitInfo& w) -> bool {
            const int buf = q_use & 1;
            const uint32_t par = (q_use >> 1) & 1;
            ++q_use;
            const int r_first = (warp % 8) * 16;
            const int gi_first = (2 * w.qp + u) * PF_BM + r_first;
            float2 cs[16];
#pragma unroll
            for (int r = 0; r < 16; ++r) cs[r] = __ldg(p.table + (size_t)min(gi_first + r, p.S - 1) * (PF_D / 2) + lane);
            if (!mbar_wait(smem_u32(&bar_qfull[buf][u]), par, &s_abort)) return false;
            const uint32_t tile = sQ + (buf * 2 + u) * PF_TILE_BYTES + r_first * 128 + (lane & 3) * 4;
            const uint32_t chunk = (uint32_t)lane >> 2;
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
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_qrot[buf][u]));
            return true;
        };
        int it;
        UnitInfo w;
        find_unit(0, it, w);
        if (it >= 0) ok = rotate_q(w);
        while (ok && it >= 0) {
            const int nt = w.n_t[u];
            const int b = w.b, h = w.h;
            const int i0 = (2 * w.qp + u) * PF_BM;
            const int gi = i0 + row;

            float m_ref = 0.f;         // exponent reference, raw score units (the same in both threads of a row)
            float l_run = 0.f;         // this thread's half of the row sum
            const int row_last = p.causal ? min(p.S - 1, gi + p.position_offset) : p.S - 1;
            const int tile_free_last = p.causal ? min(p.S - 1, i0 + p.position_offset) : p.S - 1;   // no mask needed up to here

            for (int j = 0; j < nt; ++j) {
                ok = mbar_wait(smem_u32(&bar_s[u]), (tiles_done + j) & 1, &s_abort);
                if (!ok) break;
                tc::fence_after_sync();
                const int j0 = j * PF_BN + hf * 64;             // first key of this thread's 64 columns
                const bool need_mask = (j0 + 63) > tile_free_last;

                // one pass over this thread's 64 columns: P = exp2(S * scale_log2 - m_ref * scale_log2) -> TMEM, with
                // the load of the next 16 columns in flight while the current 16 are processed
                auto half_pass = [&](float mneg, bool first_store_needs_pv) {
                    uint64_t sum2 = 0;   // (0.f, 0.f)
                    const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2), mneg2 = pack_f32x2(mneg, mneg);
                    uint32_t r0[16], r1[16], pk[8];
                    auto chunk = [&](uint32_t (&r)[16], int c) {
                        if (need_mask) softmax_chunk16<true>(r, pk, scale2, mneg2, j0 + c * 16, row_last, sum2);
                        else softmax_chunk16<false>(r, pk, scale2, mneg2, j0 + c * 16, row_last, sum2);
                    };
                    tc::ld16(tS + 0, r0);
                    tc::wait_ld(r0);
                    tc::ld16(tS + 16, r1);
                    chunk(r0, 0);
                    // P(j-1) is still being read by its P V until bar_pv says otherwise
                    bool good = true;
                    if (first_store_needs_pv) {
                        good = mbar_wait(smem_u32(&bar_pv[u]), (tiles_done + j - 1) & 1, &s_abort);
                        tc::fence_after_sync();
                    }
                    tc::st8(tP + 0, pk);
                    tc::wait_ld(r1);
                    tc::ld16(tS + 32, r0);
                    chunk(r1, 1);
                    tc::st8(tP + 8, pk);
                    tc::wait_ld(r0);
                    tc::ld16(tS + 48, r1);
                    chunk(r0, 2);
                    tc::st8(tP + 16, pk);
                    tc::wait_ld(r1);
                    chunk(r1, 3);
                    tc::st8(tP + 24, pk);
                    float s0, s1;
                    unpack_f32x2(sum2, s0, s1);
                    return good ? s0 + s1 : NAN;
                };

                // The exponent reference starts at 0 and moves only when it has to: p = 2^(s*c - ref) may be
                // anywhere in [2^-64, 2^64] without any loss (bf16 and fp32 keep their relative precision over
                // that range), so for ordinary score magnitudes there is never a second pass or an O rescale.
                float lsum = half_pass(-m_ref * p.scale_log2, tiles_done + j > 0);
                if (s_abort) { ok = false; break; }
                const bool over = !(lsum <= 0x1p64f) || (j == 0 && hf == 0 && lsum < 0x1p-64f);
                if (named_bar_or(pair_bar, 64, over)) {
                    // rare, and taken by both warps of these rows together: move the reference to the true row
                    // maximum, rescale O and l, redo the step.
                    float hmax = -INFINITY;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t r[16];
                        tc::ld16(tS + c * 16, r);
                        tc::wait_ld(r);
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (!need_mask || j0 + c * 16 + i <= row_last) hmax = fmaxf(hmax, __uint_as_float(r[i]));
                    }
                    s_xchg[u][hf][row] = hmax;
                    named_bar_sync(pair_bar, 64);
                    const float tmax = fmaxf(hmax, s_xchg[u][hf ^ 1][row]);
                    const float m_new = j == 0 ? tmax : fmaxf(m_ref, tmax);   // the first step may also move it down
                    const float m_upd = m_new == -INFINITY ? m_ref : m_new;
                    if (j > 0) {
                        const float alpha = ex2((m_ref - m_upd) * p.scale_log2);
                        l_run *= alpha;
                        uint32_t ro[32];           // this thread's 32 of the 64 O columns
                        tc::ld32(tO, ro);
                        tc::wait_ld(ro);
#pragma unroll
                        for (int i = 0; i < 32; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * alpha);
                        tc::st32(tO, ro);
                    }
                    m_ref = m_upd;
                    lsum = half_pass(-m_ref * p.scale_log2, false);
                    named_bar_sync(pair_bar, 64);      // the exchange slots may be written again
                }
                l_run += lsum;
                tc::wait_st();
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_p[u]));
            }
            if (!ok) break;
            tiles_done += nt;

            // The next unit's Q tile is rotated BEFORE this unit's epilogue: the MMA warp needs it to start the
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
            s_xchg[u][hf][row] = l_run;
            named_bar_sync(pair_bar, 64);
            const float l_row = l_run + s_xchg[u][hf ^ 1][row];
            const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
            __nv_bfloat16* dst = p.out + (((size_t)b * p.S + gi) * p.Hq + h) * PF_D + hf * 32;
            uint32_t ro[32];
            tc::ld32(tO, ro);
            tc::wait_ld(ro);
            // the next unit's first P V overwrites O only after this group's next P arrive, which follows these loads
            if (gi < p.S) {
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    uint4 o4;
                    o4.x = pack_bf16(__uint_as_float(ro[v * 8 + 0]) * inv, __uint_as_float(ro[v * 8 + 1]) * inv);
                    o4.y = pack_bf16(__uint_as_float(ro[v * 8 + 2]) * inv, __uint_as_float(ro[v * 8 + 3]) * inv);
                    o4.z = pack_bf16(__uint_as_float(ro[v * 8 + 4]) * inv, __uint_as_float(ro[v * 8 + 5]) * inv);
                    o4.w = pack_bf16(__uint_as_float(ro[v * 8 + 6]) * inv, __uint_as_float(ro[v * 8 + 7]) * inv);
                    *reinterpret_cast<uint4*>(dst + v * 8) = o4;
                }
#ifndef BN_TIMELINE
                if (p.lse && hf == 0)
                    p.lse[((size_t)b * p.Hq + h) * p.S + gi] =
                        l_row > 0.f ? (m_ref * p.scale_log2 + log2f(l_row)) * PF_LN2 : -INFINITY;
#endif
            }
            it = it_next;
            w = w_next;
        }
        // a warp that gives up (a bounded wait ran out) releases its partner, which may be waiting at the named barrier
        if (!ok) named_bar_arrive(pair_bar, 64);
    }

    // common exit: everybody arrives here (all waits are bounded), then TMEM is freed
    tc::fence_before_sync();
    __syncthreads();
    if (tid == 0 && s_abort) atomicExch(p.error_word, BN_ERR_TIMEOUT);
    if (warp == 16) {
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
    if (flags & ~(BN_PREFILL_REUSE_ROTATED_K | BN_PREFILL_SINGLE_TILE_KERNEL))
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
        rope_k_kernel<<<dim3((S + RK_POS - 1) / RK_POS, B), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(k), krot, table, B, S, Hkv, theta,
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

// C (M,N) bf16 = A (M,K) bf16 @ Bt (N,K)^T bf16, fp32 accumulation in tensor memory, for sm_100a.
//
// This is the projection GEMM of the attention layer (q/k/v/o_proj: `hidden_states @ W`,
// mygrad/llama/llama_layers.py:157-159,186; reference operator op_mm, src/ops/op_mm.cuh:39-57) on bf16 operands
// with the weight stored transposed, (out_features, in_features), so that both operands are K-major: the same
// operand form as Q K^T in the prefill kernel.
//
// Persistent kernel, one CTA per SM, 192 threads:
//   warps 0-3  epilogue: TMEM -> registers -> bf16 -> global (thread = output row = TMEM lane)
//   warp 4     MMA issuer: tcgen05.mma.cta_group::1.kind::f16, 128 x 256 x 16 per instruction
//   warp 5     TMA producer: A tile 128 x 64 and Bt tile 256 x 64 per stage (48 KB), 4-stage mbarrier ring
// Output tile 128 x 256; the fp32 accumulator (256 TMEM columns) is double buffered, so the epilogue of one tile
// runs under the main loop of the next.  Tiles are walked N-panel by N-panel with M fastest, so the CTAs that run
// together share their Bt panel in L2.  Edges: TMA zero-fills loads beyond M, N, K; stores are bounds-checked.
// Epilogue variants: plain (C = the accumulator as bf16) and SwiGLU (`MLP.__call__`, mygrad/llama/llama_layers.py:217-232,
// SiLU as op_silu.cuh:7-15): Bt holds, per 256-row tile, 128 rows of the gate weight followed by the 128 rows of the up
// weight for the same intermediate indices, so one thread finds gate and up of an output element in the same
// accumulator row and writes silu(gate) * up -- the two GEMMs, the activation and the product in one launch.
// Every mbarrier wait is bounded; on expiry the kernel raises the caller's error word, frees TMEM and returns.
#include "common.cuh"
#include "ptx.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace bn {

using namespace ptx;

constexpr int GM_BM = 128, GM_BK = 64;
constexpr int GM_A_BYTES = GM_BM * GM_BK * 2;          // 16384
constexpr int GM_THREADS = 192;
// per N-tile width BN (256: the throughput shape; 64: many small tiles for M <= 128, where the weight stream has to
// be spread over all SMs): ring depth, bytes, TMEM columns (two accumulators of BN columns, a power of two >= 32)
template <int BN> struct GemmShape {
    static constexpr int NSTAGE = BN == 256 ? 4 : 8;
    static constexpr int B_BYTES = BN * GM_BK * 2;
    static constexpr int STAGE_BYTES = GM_A_BYTES + B_BYTES;
    static constexpr int SMEM_BYTES = 1024 + NSTAGE * STAGE_BYTES;
    static constexpr uint32_t TMEM_COLS = 2 * BN;
};

// EPI_QKV: the q, k and v projections of the layer as ONE product with the concatenated weight; the epilogue sends
// each 32-column piece where it belongs (below)
struct QkvEpilogue {
    __nv_bfloat16* q;            // (tokens, NQ) as projected (the attention kernel rotates Q itself)
    __nv_bfloat16* krot;         // (tokens, NK) rotated K, the attention kernel's operand
    __nv_bfloat16* v;            // (tokens, NK)
    const float2* table;         // [S][32] cos/sin of position s + position_offset
    int* kmax2;                  // [B][Hkv][key tiles of 128]: largest |rotated k|^2 as float bits (atomic max)
    __nv_bfloat16* pool;         // paged cache (may be null): pool[page][kv_head][K|V][16][64]
    const int32_t* page_table;   // (B, max_pages)
    long long pool_pages;
    int max_pages, S, NQ, NK, Hkv, n_ktiles, position_offset;
};

constexpr int EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_PARTIAL = 2, EPI_QKV = 3;

struct GemmParams {
    __nv_bfloat16* c;
    int* error_word;       // optional
    int M, N, K;           // N = rows of Bt
    int n_out;             // columns of C: N (plain) or the intermediate size (SwiGLU)
    float* partial;        // EPI_PARTIAL: [split][M][N] fp32
    int splits, k_per_split;   // EPI_PARTIAL: K steps are cut into `splits` ranges of k_per_split steps
    QkvEpilogue qkv;       // EPI_QKV
};



template <int EPI, int GM_BN>
__global__ void __launch_bounds__(GM_THREADS, 1)
gemm_bf16_nt_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmParams p) {
    constexpr int GM_NSTAGE = GemmShape<GM_BN>::NSTAGE, GM_STAGE_BYTES = GemmShape<GM_BN>::STAGE_BYTES;
    constexpr uint32_t GM_TMEM_COLS = GemmShape<GM_BN>::TMEM_COLS;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[GM_NSTAGE], bar_empty[GM_NSTAGE], bar_acc_full[2], bar_acc_empty[2];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int tiles_m = (p.M + GM_BM - 1) / GM_BM, tiles_n = (p.N + GM_BN - 1) / GM_BN;
    const int k_steps_all = (p.K + GM_BK - 1) / GM_BK;
    // a work item is an output tile, or (EPI_PARTIAL) a tile and one range of the K steps
    const int splits = EPI == EPI_PARTIAL ? p.splits : 1;
    const int n_tiles = tiles_m * tiles_n * splits;
    auto k_range = [&](int t, int& ks0, int& ks1) {
        if (EPI == EPI_PARTIAL) {
            ks0 = (t / (tiles_m * tiles_n)) * p.k_per_split;
            ks1 = min(k_steps_all, ks0 + p.k_per_split);
        } else {
            ks0 = 0;
            ks1 = k_steps_all;
        }
    };

    if (tid == 0) {
        for (int s = 0; s < GM_NSTAGE; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&bar_acc_full[i]), 1);
            mbar_init(smem_u32(&bar_acc_empty[i]), 4);      // one arrive per epilogue warp
        }
        s_abort = 0;
        fence_mbar_init();
    }
    if (warp == 4) {
        tc::tmem_alloc(smem_u32(&s_tmem_base), GM_TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = s_tmem_base;

    if (warp == 5) {
        // ---------------------------------------------------------- TMA producer
        if (lane == 0) {
            prefetch_tensormap(&tmap_a);
            prefetch_tensormap(&tmap_b);
            uint32_t it = 0;      // ring steps issued
            bool ok = true;
            for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x) {
                const int m0 = (t % tiles_m) * GM_BM, n0 = ((t / tiles_m) % tiles_n) * GM_BN;
                int ks0, ks1;
                k_range(t, ks0, ks1);
                for (int ks = ks0; ks < ks1; ++ks, ++it) {
                    const int stage = it % GM_NSTAGE;
                    ok = mbar_wait(smem_u32(&bar_empty[stage]), ((it / GM_NSTAGE) & 1u) ^ 1u, &s_abort);
                    if (!ok) break;
                    const uint32_t sA = smem0 + stage * GM_STAGE_BYTES, sB = sA + GM_A_BYTES;
                    mbar_arrive_expect_tx(smem_u32(&bar_full[stage]), GM_STAGE_BYTES);
                    tma_load_2d(sA, &tmap_a, ks * GM_BK, m0, smem_u32(&bar_full[stage]));
                    tma_load_2d(sB, &tmap_b, ks * GM_BK, n0, smem_u32(&bar_full[stage]));
                }
            }
        }
    } else if (warp == 4) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t IDESC = tc::idesc_bf16(GM_BM, GM_BN, 0);
        const uint64_t dZero = tc::smem_desc_sw128(0);   // descriptor = this + (address >> 4)
        uint32_t it = 0, local = 0;
        bool ok = true;
        for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x, ++local) {
            const uint32_t acc = local & 1u;
            // the epilogue must have drained this accumulator (two tiles ago)
            ok = mbar_wait(smem_u32(&bar_acc_empty[acc]), ((local >> 1) & 1u) ^ 1u, &s_abort);
            if (!ok) break;
            tc::fence_after_sync();
            int ks0, ks1;
            k_range(t, ks0, ks1);
            for (int ks = ks0; ks < ks1; ++ks, ++it) {
                const int stage = it % GM_NSTAGE;
                ok = mbar_wait(smem_u32(&bar_full[stage]), (it / GM_NSTAGE) & 1u, &s_abort);
                if (!ok) break;
                if (elect_one()) {
                    tc::fence_after_sync();
                    const uint32_t sA = smem0 + stage * GM_STAGE_BYTES, sB = sA + GM_A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < GM_BK / 16; ++kk)
                        tc::mma_ss(tmem + acc * GM_BN, dZero + (uint64_t)((sA >> 4) + kk * 2),
                                   dZero + (uint64_t)((sB >> 4) + kk * 2), IDESC, (ks > ks0) || (kk > 0));
                    tc::commit(smem_u32(&bar_empty[stage]));                       // the stage may be refilled
                    if (ks == ks1 - 1) tc::commit(smem_u32(&bar_acc_full[acc]));  // the tile is complete
                }
                __syncwarp();
            }
        }
    } else {
        // ------------------------------------------------------ epilogue (warps 0..3)
        const int row = tid;                                   // TMEM lane = output row inside the tile
        const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
        uint32_t local = 0;
        bool ok = true;
        for (int t = blockIdx.x; ok && t < n_tiles; t += gridDim.x, ++local) {
            const uint32_t acc = local & 1u;
            const int m0 = (t % tiles_m) * GM_BM, n0 = ((t / tiles_m) % tiles_n) * GM_BN;
            ok = mbar_wait(smem_u32(&bar_acc_full[acc]), (local >> 1) & 1u, &s_abort);
            if (!ok) break;
            tc::fence_after_sync();
            const int gm = m0 + row;
            if (EPI == EPI_PLAIN) {
                __nv_bfloat16* crow = p.c + (size_t)gm * p.n_out + n0;
#pragma unroll 1
                for (int c = 0; c < GM_BN / 32; ++c) {
                    uint32_t r[32];
                    tc::ld32(tmem + lane_base + acc * GM_BN + c * 32, r);
                    tc::wait_ld(r);
                    if (gm < p.M) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            const int col = n0 + c * 32 + v * 8;
                            if (col < p.n_out) {    // a multiple of 8: a group of 8 columns is all in or all out
                                uint4 o4;
                                o4.x = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                                o4.y = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                                o4.z = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                                o4.w = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
                                *reinterpret_cast<uint4*>(crow + c * 32 + v * 8) = o4;
                            }
                        }
                    }
                }
            } else if (EPI == EPI_QKV) {
                // Columns [0, NQ) are Q: written as they are.  [NQ, NQ + NK) are K: rotated at the row's position
                // (pairs (2i, 2i+1) of each 64-wide head, src/ops/op_rope.cuh:55-99, from the fp32 accumulators:
                // one rounding instead of two), written as the attention kernel's K operand AND into the row's page
                // of the cache, with the largest squared norm per (sequence, KV head, 128-key tile) kept for that
                // kernel's bound on the scores.  The rest is V: written to the V operand and into the cache.
                // A 32-column piece is half a head, so a piece never straddles two of these regions or two heads.
                const QkvEpilogue& e = p.qkv;
                const bool live = gm < p.M;
                const int b = live ? gm / e.S : 0, srow = live ? gm - b * e.S : 0;
                const int pos = srow + e.position_offset;
                long long page = -1;
                if (e.pool && live && n0 + GM_BN > e.NQ) {
                    const int lp = pos / BN_PAGE_TOKENS;
                    if (lp < e.max_pages) page = e.page_table[(size_t)b * e.max_pages + lp];
                    if (page >= e.pool_pages) page = -1;
                }
                const int slot = pos % BN_PAGE_TOKENS;
                const int key = live ? b * e.n_ktiles + srow / 128 : -1;         // which norm slot this row feeds
                const bool same_key = __all_sync(0xffffffffu, key == __shfl_sync(0xffffffffu, key, 0) && key >= 0);
                float head_n2 = 0.f;
#pragma unroll 1
                for (int c = 0; c < GM_BN / 32; ++c) {
                    uint32_t r[32];
                    tc::ld32(tmem + lane_base + acc * GM_BN + c * 32, r);
                    tc::wait_ld(r);
                    const int col = n0 + c * 32;
                    if (col >= p.N) continue;                 // (uniform) beyond the concatenated weight
                    uint4 o4[4];
                    if (col < e.NQ || col >= e.NQ + e.NK) {   // Q or V: plain rounding
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            o4[v].x = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                            o4[v].y = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                            o4[v].z = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                            o4[v].w = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
                        }
                        if (live) {
                            if (col < e.NQ) {
                                uint4* dst = reinterpret_cast<uint4*>(e.q + (size_t)gm * e.NQ + col);
#pragma unroll
                                for (int v = 0; v < 4; ++v) dst[v] = o4[v];
                            } else {
                                const int vc = col - e.NQ - e.NK;
                                uint4* dst = reinterpret_cast<uint4*>(e.v + (size_t)gm * e.NK + vc);
#pragma unroll
                                for (int v = 0; v < 4; ++v) dst[v] = o4[v];
                                if (page >= 0) {
                                    uint4* pd = reinterpret_cast<uint4*>(
                                        e.pool + (((page * e.Hkv + vc / 64) * 2 + 1) * BN_PAGE_TOKENS + slot) * 64 + vc % 64);
#pragma unroll
                                    for (int v = 0; v < 4; ++v) pd[v] = o4[v];
                                }
                            }
                        }
                    } else {                                   // K: rotate, round, norms
                        const int kc = col - e.NQ;             // column inside K; kc % 64 is 0 or 32
                        const float2* cs = e.table + (size_t)srow * 32 + (kc % 64) / 2;
                        uint32_t w[16];
                        float n2 = 0.f;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float2 t2 = live ? __ldg(cs + i) : make_float2(1.f, 0.f);
                            const float x0 = __uint_as_float(r[2 * i]), x1 = __uint_as_float(r[2 * i + 1]);
                            w[i] = pack_bf16(x0 * t2.x - x1 * t2.y, x0 * t2.y + x1 * t2.x);
                            const float y0 = bf16_lo(w[i]), y1 = bf16_hi(w[i]);
                            n2 = fmaf(y0, y0, fmaf(y1, y1, n2));
                        }
#pragma unroll
                        for (int v = 0; v < 4; ++v) o4[v] = make_uint4(w[v * 4], w[v * 4 + 1], w[v * 4 + 2], w[v * 4 + 3]);
                        if (live) {
                            uint4* dst = reinterpret_cast<uint4*>(e.krot + (size_t)gm * e.NK + kc);
#pragma unroll
                            for (int v = 0; v < 4; ++v) dst[v] = o4[v];
                            if (page >= 0) {
                                uint4* pd = reinterpret_cast<uint4*>(
                                    e.pool + (((page * e.Hkv + kc / 64) * 2 + 0) * BN_PAGE_TOKENS + slot) * 64 + kc % 64);
#pragma unroll
                                for (int v = 0; v < 4; ++v) pd[v] = o4[v];
                            }
                        }
                        head_n2 += n2;
                        if (kc % 64) {                         // second half of the head: its norm is complete
                            // a NaN or an infinity must read as "unbounded": their bit patterns are above every finite float's
                            int bits = live ? (head_n2 == head_n2 ? __float_as_int(head_n2) : 0x7fffffff) : 0;
                            const int hh = kc / 64;
                            if (same_key) {
                                bits = __reduce_max_sync(0xffffffffu, bits);
                                if (lane == 0) atomicMax(e.kmax2 + ((size_t)b * e.Hkv + hh) * e.n_ktiles + srow / 128, bits);
                            } else if (live) {
                                atomicMax(e.kmax2 + ((size_t)b * e.Hkv + hh) * e.n_ktiles + srow / 128, bits);
                            }
                            head_n2 = 0.f;
                        }
                    }
                }
            } else if (EPI == EPI_PARTIAL) {
                // the fp32 partial sum of this K range; the ranges are added in order by the reduce kernel
                float* prow = p.partial + ((size_t)(t / (tiles_m * tiles_n)) * p.M + gm) * p.N + n0;
#pragma unroll 1
                for (int c = 0; c < GM_BN / 32; ++c) {
                    uint32_t r[32];
                    tc::ld32(tmem + lane_base + acc * GM_BN + c * 32, r);
                    tc::wait_ld(r);
                    if (gm < p.M) {
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            const int col = n0 + c * 32 + v * 4;
                            if (col < p.N)          // N is a multiple of 8
                                *reinterpret_cast<float4*>(prow + c * 32 + v * 4) =
                                    make_float4(__uint_as_float(r[v * 4]), __uint_as_float(r[v * 4 + 1]),
                                                __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3]));
                        }
                    }
                }
            } else {
                // accumulator columns [0,128) = gate, [128,256) = up, of intermediate indices n0/2 .. n0/2 + 127
                const int i0 = n0 / 2;
                __nv_bfloat16* crow = p.c + (size_t)gm * p.n_out + i0;
#pragma unroll 1
                for (int c = 0; c < GM_BN / 64; ++c) {
                    uint32_t g[32], u[32];
                    tc::ld32(tmem + lane_base + acc * GM_BN + c * 32, g);
                    tc::ld32(tmem + lane_base + acc * GM_BN + GM_BN / 2 + c * 32, u);
                    tc::wait_ld(g);
                    tc::wait_ld(u);
                    if (gm < p.M) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            const int col = i0 + c * 32 + v * 8;
                            if (col < p.n_out) {
                                float h[8];
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    const float gv = __uint_as_float(g[v * 8 + e]);
                                    // silu(g) * up, silu(g) = g / (1 + exp(-g))
                                    h[e] = __fdividef(gv, 1.f + __expf(-gv)) * __uint_as_float(u[v * 8 + e]);
                                }
                                uint4 o4;
                                o4.x = pack_bf16(h[0], h[1]);
                                o4.y = pack_bf16(h[2], h[3]);
                                o4.z = pack_bf16(h[4], h[5]);
                                o4.w = pack_bf16(h[6], h[7]);
                                *reinterpret_cast<uint4*>(crow + c * 32 + v * 8) = o4;
                            }
                        }
                    }
                }
            }
            // this warp has read its lanes of the accumulator
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[acc]));
        }
    }

    // common exit: everybody arrives here (all waits are bounded), then TMEM is freed
    tc::fence_before_sync();
    __syncthreads();
    if (tid == 0 && s_abort && p.error_word) atomicExch(p.error_word, BN_ERR_TIMEOUT);
    if (warp == 4) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem, GM_TMEM_COLS);
    }
}

}  // namespace bn

using namespace bn;

// sum of the split-K partials, in split order (deterministic), rounded once to bf16
__global__ void __launch_bounds__(256)
gemm_splitk_reduce_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ c, long long mn4, int splits) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;     // one group of 4 outputs
    if (i >= mn4) return;
    const float4* p4 = reinterpret_cast<const float4*>(partial);
    float4 acc = __ldcg(p4 + i);
    for (int s = 1; s < splits; ++s) {
        const float4 v = __ldcg(p4 + (long long)s * mn4 + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<uint2*>(c)[i] = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
}

// how a small-M product is cut: 64-wide N tiles, and the K steps into `splits` ranges so that about one work item
// per SM exists; never more than 8 ranges (the partial sums are extra traffic) nor ranges shorter than 4 K steps
static void splitk_plan(int M, int N, int K, int sms, int* splits, int* k_per_split) {
    const long long tiles = (long long)((M + GM_BM - 1) / GM_BM) * ((N + 63) / 64);
    const int k_steps = (K + GM_BK - 1) / GM_BK;
    long long want = tiles >= sms ? 1 : (sms + tiles - 1) / tiles;
    if (want > 8) want = 8;
    if (want > k_steps / 4) want = k_steps / 4 > 0 ? k_steps / 4 : 1;
    const int per = (int)((k_steps + want - 1) / want);
    *k_per_split = per;
    *splits = (k_steps + per - 1) / per;
}

template <int EPI, int BN>
static int gemm_configure(int dev) {
    static thread_local int configured_dev = -1;
    if (configured_dev == dev) return BN_OK;
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_nt_kernel<EPI, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GemmShape<BN>::SMEM_BYTES);
    if (e != cudaSuccess) return fail(BN_ERR_CUDA, "cudaFuncSetAttribute(gemm): %s", cudaGetErrorString(e));
    configured_dev = dev;
    return BN_OK;
}

static int gemm_launch(const void* a, const void* bt, void* c, int M, int N, int K, int n_out, int epi, int* error_word,
                       bn_stream_t stream, const char* what, float* partial = nullptr, int splits = 1,
                       int k_per_split = 0, const QkvEpilogue* qkv = nullptr) {
    if (!a || !bt || !c) return fail(BN_ERR_INVALID_ARG, "%s: null pointer", what);
    if (M < 0 || N < 0 || K < 0 || n_out < 0) return fail(BN_ERR_INVALID_ARG, "%s: bad shape M=%d N=%d K=%d", what, M, N, K);
    if (n_out % 8 || K % 8)
        return fail(BN_ERR_UNSUPPORTED, "%s: N=%d and K=%d must be multiples of 8 (16-byte rows)", what, n_out, K);
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(bt) | reinterpret_cast<uintptr_t>(c)) & 15)
        return fail(BN_ERR_INVALID_ARG, "%s: a/bt/c must be 16-byte aligned", what);
    if (int rc = require_sm100()) return rc;
    if (M == 0 || n_out == 0) return BN_OK;
    if (K == 0) {
        cudaError_t e = cudaMemsetAsync(c, 0, (size_t)M * n_out * 2, as_stream(stream));
        return e == cudaSuccess ? BN_OK : fail(BN_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    }
    const int bn = epi == EPI_PARTIAL ? 64 : 256;
    CUtensorMap tmap_a, tmap_b;
    {
        const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M}, strides[1] = {(uint64_t)K * 2};
        const uint32_t box[2] = {GM_BK, GM_BM};
        if (int rc = make_tensor_map(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, dims, strides, box,
                                     CU_TENSOR_MAP_SWIZZLE_128B))
            return rc;
    }
    {
        const uint64_t dims[2] = {(uint64_t)K, (uint64_t)N}, strides[1] = {(uint64_t)K * 2};
        const uint32_t box[2] = {GM_BK, (uint32_t)bn};
        if (int rc = make_tensor_map(&tmap_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, bt, dims, strides, box,
                                     CU_TENSOR_MAP_SWIZZLE_128B))
            return rc;
    }
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long n_items = (long long)((M + GM_BM - 1) / GM_BM) * ((N + bn - 1) / bn) * splits;
    GemmParams p{static_cast<__nv_bfloat16*>(c), error_word, M, N, K, n_out, partial, splits, k_per_split, QkvEpilogue{}};
    if (qkv) p.qkv = *qkv;
    const unsigned grid = (unsigned)(n_items < sms ? n_items : sms);
    cudaStream_t st = as_stream(stream);
    if (epi == EPI_PLAIN) {
        if (int rc = gemm_configure<EPI_PLAIN, 256>(dev)) return rc;
        gemm_bf16_nt_kernel<EPI_PLAIN, 256><<<grid, GM_THREADS, GemmShape<256>::SMEM_BYTES, st>>>(tmap_a, tmap_b, p);
    } else if (epi == EPI_SWIGLU) {
        if (int rc = gemm_configure<EPI_SWIGLU, 256>(dev)) return rc;
        gemm_bf16_nt_kernel<EPI_SWIGLU, 256><<<grid, GM_THREADS, GemmShape<256>::SMEM_BYTES, st>>>(tmap_a, tmap_b, p);
    } else if (epi == EPI_QKV) {
        if (int rc = gemm_configure<EPI_QKV, 256>(dev)) return rc;
        gemm_bf16_nt_kernel<EPI_QKV, 256><<<grid, GM_THREADS, GemmShape<256>::SMEM_BYTES, st>>>(tmap_a, tmap_b, p);
    } else {
        if (int rc = gemm_configure<EPI_PARTIAL, 64>(dev)) return rc;
        gemm_bf16_nt_kernel<EPI_PARTIAL, 64><<<grid, GM_THREADS, GemmShape<64>::SMEM_BYTES, st>>>(tmap_a, tmap_b, p);
        if (int rc = launch_status(what)) return rc;
        const long long mn4 = (long long)M * N / 4;
        gemm_splitk_reduce_kernel<<<(unsigned)((mn4 + 255) / 256), 256, 0, st>>>(partial, static_cast<__nv_bfloat16*>(c),
                                                                             mn4, splits);
    }
    return launch_status(what);
}

extern "C" int bn_gemm_bf16_nt(const void* a, const void* bt, void* c, int M, int N, int K, int* error_word,
                               bn_stream_t stream) {
    return gemm_launch(a, bt, c, M, N, K, N, EPI_PLAIN, error_word, stream, "bn_gemm_bf16_nt");
}

extern "C" int bn_gemm_swiglu_bf16_nt(const void* x, const void* gate_up_t, void* h, int M, int inter, int K,
                                      int* error_word, bn_stream_t stream) {
    if (inter < 0) return fail(BN_ERR_INVALID_ARG, "bn_gemm_swiglu_bf16_nt: bad shape inter=%d", inter);
    const int n_rows = (inter + 127) / 128 * 256;      // rows of the packed gate/up weight
    return gemm_launch(x, gate_up_t, h, M, n_rows, K, inter, EPI_SWIGLU, error_word, stream, "bn_gemm_swiglu_bf16_nt");
}

extern "C" size_t bn_gemm_bf16_nt_small_m_workspace_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    int dev = 0, sms = 0, splits = 1, per = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    splitk_plan(M, N, K, sms, &splits, &per);
    return (size_t)splits * M * N * sizeof(float);
}

extern "C" int bn_gemm_bf16_nt_small_m(const void* a, const void* bt, void* c, int M, int N, int K, void* workspace,
                                       size_t workspace_bytes, int* error_word, bn_stream_t stream) {
    if (M > 0 && N > 0 && K > 0) {
        if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15))
            return fail(BN_ERR_WORKSPACE, "bn_gemm_bf16_nt_small_m: workspace missing or not 16-byte aligned");
        int dev = 0, sms = 0, splits = 1, per = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        splitk_plan(M, N, K, sms, &splits, &per);
        if (workspace_bytes < (size_t)splits * M * N * sizeof(float))
            return fail(BN_ERR_WORKSPACE, "bn_gemm_bf16_nt_small_m: workspace of %zu bytes is too small", workspace_bytes);
        return gemm_launch(a, bt, c, M, N, K, N, EPI_PARTIAL, error_word, stream, "bn_gemm_bf16_nt_small_m",
                           static_cast<float*>(workspace), splits, per);
    }
    return gemm_launch(a, bt, c, M, N, K, N, EPI_PARTIAL, error_word, stream, "bn_gemm_bf16_nt_small_m");
}

extern "C" int bn_gemm_qkv_rope_bf16(const void* x, const void* wqkv_t, void* q_out, void* v_out, int B, int S, int hidden,
                                     int Hq, int Hkv, int D, int position_offset, void* prefill_workspace,
                                     size_t prefill_workspace_bytes, void* pool, int64_t pool_pages,
                                     const int32_t* page_table, int max_pages, int* error_word, bn_stream_t stream) {
    const char* what = "bn_gemm_qkv_rope_bf16";
    if (!x || !wqkv_t || !q_out || !v_out || !prefill_workspace) return fail(BN_ERR_INVALID_ARG, "%s: null pointer", what);
    if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || hidden <= 0 || position_offset < 0)
        return fail(BN_ERR_INVALID_ARG, "%s: bad shape B=%d S=%d Hq=%d Hkv=%d hidden=%d", what, B, S, Hq, Hkv, hidden);
    if (D != 64) return fail(BN_ERR_UNSUPPORTED, "%s: head_dim=%d (64 supported)", what, D);
    if (pool && (!page_table || max_pages <= 0 || pool_pages <= 0))
        return fail(BN_ERR_INVALID_ARG, "%s: a cache pool needs its page table", what);
    if ((reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(v_out) | reinterpret_cast<uintptr_t>(pool)) & 15)
        return fail(BN_ERR_INVALID_ARG, "%s: q/v/pool must be 16-byte aligned", what);
    size_t off_table = 0, off_kmax2 = 0, off_krot = 0, total = 0;
    prefill_bf16_workspace_layout(B, S, Hkv, &off_table, &off_kmax2, &off_krot, &total);
    if (prefill_workspace_bytes < total)
        return fail(BN_ERR_WORKSPACE, "%s: workspace of %zu bytes given, %zu needed (bn_attn_prefill_bf16_workspace_bytes)",
                    what, prefill_workspace_bytes, total);
    if (reinterpret_cast<uintptr_t>(prefill_workspace) & 255)
        return fail(BN_ERR_INVALID_ARG, "%s: workspace must be 256-byte aligned", what);
    uint8_t* ws = static_cast<uint8_t*>(prefill_workspace);
    // the norm maxima are taken with atomics: clear them first (a few KB)
    cudaError_t ce = cudaMemsetAsync(ws + off_kmax2, 0, off_krot - off_kmax2, as_stream(stream));
    if (ce != cudaSuccess) return fail(BN_ERR_CUDA, "%s: cudaMemsetAsync: %s", what, cudaGetErrorString(ce));
    QkvEpilogue e;
    e.q = static_cast<__nv_bfloat16*>(q_out);
    e.krot = reinterpret_cast<__nv_bfloat16*>(ws + off_krot);
    e.v = static_cast<__nv_bfloat16*>(v_out);
    e.table = reinterpret_cast<const float2*>(ws + off_table);
    e.kmax2 = reinterpret_cast<int*>(ws + off_kmax2);
    e.pool = static_cast<__nv_bfloat16*>(pool);
    e.page_table = page_table;
    e.pool_pages = pool_pages;
    e.max_pages = max_pages;
    e.S = S; e.NQ = Hq * D; e.NK = Hkv * D; e.Hkv = Hkv; e.n_ktiles = (S + 127) / 128; e.position_offset = position_offset;
    const int N = (Hq + 2 * Hkv) * D;
    return gemm_launch(x, wqkv_t, q_out, B * S, N, hidden, N, EPI_QKV, error_word, stream, what, nullptr, 1, 0, &e);
}

// Single-token decode attention over the paged bf16 KV cache (HBM-bound).
//
// Decode semantics follow the reference's generate loop, where the new token's
// output is the last row of an attention over everything before it
// (mygrad/llama/llama_model.py:136-144); here the earlier keys/values come from
// the cache instead of being recomputed.
//
// Design (one persistent CTA per SM):
//   * Work item = (sequence, KV head, chunk of `chunk` tokens), claimed from an
//     atomic counter so that SMs stay balanced over ragged lengths.
//   * A producer warp streams the item's pages through a ring of shared-memory
//     stages with TMA tensor loads (one 4 KB box = K and V of one (page, head),
//     128-byte swizzle), completion counted on mbarriers.
//   * Four consumer warps each take two pages (32 tokens) of a stage.  All 8
//     query heads of the GQA group are served from the one K/V read:
//       S^T (16 tokens x 8 heads) = K_page (16 x 64) . Q^T (64 x 8)
//       O^T (64 dims  x 8 heads) += V_page^T (64 x 16) . P^T (16 x 8)
//     as m16n8k16 bf16 MMAs with fp32 accumulation; softmax is online, base 2.
//   * Per item the four warps merge (m, l, O) in shared memory.  A sequence cut
//     into several chunks leaves fp32 partials in scratch memory; the CTA that
//     finishes the last chunk of a (sequence, head) performs the log-sum-exp
//     combine (atomic ticket, nobody spins on another CTA).
//   * Every wait is bounded; on expiry the kernel raises the error word in the
//     scratch header and returns.
#include <math.h>
#include <stdlib.h>

#include "common.cuh"
#include "ptx.cuh"
#include "tma.cuh"

namespace bn {

using namespace ptx;

#ifndef BN_DDBG
#define BN_DDBG 0
#endif
constexpr int DEC_D = 64;
constexpr int DEC_G = 8;                    // query heads per KV head served by one MMA (n = 8)
constexpr int DEC_STAGE_TOKENS = 128;
constexpr int DEC_PAGES_PER_STAGE = DEC_STAGE_TOKENS / BN_PAGE_TOKENS;  // 8
constexpr int DEC_BOX_ROWS = 2 * BN_PAGE_TOKENS;                        // K rows then V rows
constexpr int DEC_BOX_BYTES = DEC_BOX_ROWS * DEC_D * 2;                 // 4096
constexpr int DEC_STAGE_BYTES = DEC_PAGES_PER_STAGE * DEC_BOX_BYTES;    // 32768
constexpr int DEC_NSTAGES = 6;
constexpr int DEC_CWARPS = 4;
constexpr int DEC_THREADS = (DEC_CWARPS + 1) * 32;
constexpr int DEC_SMEM_BYTES = DEC_NSTAGES * DEC_STAGE_BYTES + 1024;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct DecodeHeader {   // first 256 bytes of the scratch buffer
    int error;          // BN_ERR_TIMEOUT once a bounded wait ran out
    int work_counter;   // next work item to claim
    int done_counter;   // CTAs that ran out of work
};

struct DecodeLayout {
    size_t tickets, part_m, part_l, part_o, total;
    int max_chunks;
};

static DecodeLayout decode_layout(int B, int Hkv, int max_seq_len, int chunk) {
    DecodeLayout L;
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    L.max_chunks = max_seq_len > 0 ? (max_seq_len + chunk - 1) / chunk : 1;
    size_t bg = (size_t)B * Hkv;
    L.tickets = 256;
    L.part_m = L.tickets + up(bg * sizeof(int));
    L.part_l = L.part_m + up(bg * L.max_chunks * DEC_G * sizeof(float));
    L.part_o = L.part_l + up(bg * L.max_chunks * DEC_G * sizeof(float));
    L.total = L.part_o + up(bg * L.max_chunks * DEC_G * DEC_D * sizeof(float));
    return L;
}

static int pick_chunk(int B, int Hkv, int max_seq_len, int chunk_tokens) {
    if (chunk_tokens > 0) return chunk_tokens;
    // aim at ~8 items per SM when every sequence is at its maximum length
    long long tokens = (long long)B * Hkv * (long long)max_seq_len;
    long long c = tokens / (8 * 148) / DEC_STAGE_TOKENS * DEC_STAGE_TOKENS;
    if (c < 256) c = 256;
    if (c > 8192) c = 8192;
    return (int)c;
}

struct DecodeParams {
    const __nv_bfloat16* q;
    const int32_t* page_table;
    const int32_t* seq_lens;
    const int32_t* q_positions;
    __nv_bfloat16* out;
    float* out_f32;
    float* lse;
    DecodeHeader* hdr;
    int* tickets;
    float *part_m, *part_l, *part_o;
    int B, Hq, Hkv, n_rep, max_pages, max_seq_len, chunk, max_chunks, total_items, rope_q, debug;
    float scale_log2, theta;
};

struct StageMeta {
    int item, b, g, chunk, ntok, first, last, n_chunks, qpos;
};

__global__ void __launch_bounds__(DEC_THREADS, 1)
decode_paged_kernel(const __grid_constant__ CUtensorMap tmap, const DecodeParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[DEC_NSTAGES];
    __shared__ __align__(8) uint64_t empty_bar[DEC_NSTAGES];
    __shared__ __align__(8) uint64_t merge_bar;
    __shared__ StageMeta meta[DEC_NSTAGES];
    __shared__ float mrg_m[DEC_CWARPS][DEC_G], mrg_l[DEC_CWARPS][DEC_G];
    __shared__ float mrg_o[DEC_CWARPS][DEC_G][DEC_D + 1];
    __shared__ float s_inv_freq[DEC_D / 2];
    __shared__ int s_abort, s_ticket;

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;

    if (tid == 0) {
        for (int s = 0; s < DEC_NSTAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), DEC_CWARPS);
        }
        mbar_init(smem_u32(&merge_bar), DEC_CWARPS);
        s_abort = 0;
        s_ticket = 0;
        fence_mbar_init();
        prefetch_tensormap(&tmap);
    }
    if (tid < DEC_D / 2) s_inv_freq[tid] = rope_inv_freq(tid, DEC_D, p.theta);
    __syncthreads();

    const int BG = p.B * p.Hkv;

    if (warp == DEC_CWARPS) {
        // ------------------------------------------------------------ producer
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        while (ok) {
            int id = 0;
            if (lane == 0) id = atomicAdd(&p.hdr->work_counter, 1);
            id = __shfl_sync(0xffffffffu, id, 0);
            if (id >= p.total_items) break;
            const int c = id / BG, bg = id % BG, b = bg / p.Hkv, g = bg % p.Hkv;
            int L = p.seq_lens[b];
            L = max(0, min(L, p.max_seq_len));
            const int n_chunks = max(1, (L + p.chunk - 1) / p.chunk);
            if (c >= n_chunks) continue;
            const int t0 = c * p.chunk, t1 = min(L, t0 + p.chunk);
            const int nst = max(1, (t1 - t0 + DEC_STAGE_TOKENS - 1) / DEC_STAGE_TOKENS);
            const int qpos = p.q_positions ? p.q_positions[b] : L - 1;
            for (int s = 0; s < nst; ++s) {
                if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, &s_abort)) { ok = false; break; }
                const int ts = t0 + s * DEC_STAGE_TOKENS;
                const int ntok = max(0, min(DEC_STAGE_TOKENS, t1 - ts));
                const int npages = (ntok + BN_PAGE_TOKENS - 1) / BN_PAGE_TOKENS;
                const uint32_t fb = smem_u32(&full_bar[stage]);
                if (lane == 0) {
                    StageMeta mt{id, b, g, c, ntok, s == 0, s == nst - 1, n_chunks, qpos};
                    meta[stage] = mt;
                    if (npages > 0) mbar_arrive_expect_tx(fb, (uint32_t)npages * DEC_BOX_BYTES);
                    else mbar_arrive(fb);
                }
                __syncwarp();
                if (lane < npages) {
#if (BN_DDBG & 2)
                    const int page = (b * 61 + ts / BN_PAGE_TOKENS + lane) & 8191;
#else
                    const int page = p.page_table[(size_t)b * p.max_pages + ts / BN_PAGE_TOKENS + lane];
#endif
                    tma_load_2d(ring + stage * DEC_STAGE_BYTES + lane * DEC_BOX_BYTES, &tmap, 0,
                                (page * p.Hkv + g) * DEC_BOX_ROWS, fb);
                }
                if (++stage == DEC_NSTAGES) { stage = 0; phase ^= 1u; }
            }
        }
        if (ok && mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, &s_abort)) {
            if (lane == 0) {
                meta[stage].item = -1;   // end marker
                mbar_arrive(smem_u32(&full_bar[stage]));
            }
        }
        if (lane == 0) {
            if (s_abort) {
                atomicExch(&p.hdr->error, BN_ERR_TIMEOUT);
            } else {
                // the last CTA to run out of work re-arms the counters for the next launch
                int old = atomicAdd(&p.hdr->done_counter, 1);
                if (old == (int)gridDim.x - 1) {
                    p.hdr->work_counter = 0;
                    p.hdr->done_counter = 0;
                }
            }
        }
        return;
    }

    // --------------------------------------------------------------- consumers
    int stage = 0;
    uint32_t phase = 0, mphase = 0;
    const int hl = lane / 4;             // head (B-fragment column / S^T column pair owner)
    const int hA = 2 * (lane % 4);       // the two heads whose softmax state this thread carries
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[4][4];
    uint32_t qb[4][2] = {};
    const uint32_t mb = smem_u32(&merge_bar);

    auto group_sync = [&]() -> bool {
        __syncwarp();
        if (lane == 0) mbar_arrive(mb);
        bool ok = mbar_wait(mb, mphase, &s_abort);
        mphase ^= 1u;
        return ok;
    };

    while (true) {
        if (!mbar_wait(smem_u32(&full_bar[stage]), phase, &s_abort)) break;
        const StageMeta mt = meta[stage];
        if (mt.item < 0) break;
        const int b = mt.b, g = mt.g;

        if (mt.first) {
            // Q^T fragments (k = dims, n = heads), rotated at the query position
            const bool hv = hl < p.n_rep;
            const __nv_bfloat16* qrow = p.q + ((size_t)b * p.Hq + (size_t)g * p.n_rep + hl) * DEC_D;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
#pragma unroll
                for (int h8 = 0; h8 < 2; ++h8) {
                    const int d = kk * 16 + h8 * 8 + 2 * (lane % 4);
                    uint32_t raw = hv ? *reinterpret_cast<const uint32_t*>(qrow + d) : 0u;
                    float x0 = bf16_lo(raw), x1 = bf16_hi(raw);
                    if (p.rope_q) {
                        float angle = mt.qpos * s_inv_freq[d / 2];
                        float cos_angle = cosf(angle), sin_angle = sinf(angle);
                        float y0 = x0 * cos_angle - x1 * sin_angle;
                        float y1 = x0 * sin_angle + x1 * cos_angle;
                        x0 = y0; x1 = y1;
                    }
                    qb[kk][h8] = pack_bf16(x0, x1);
                }
            m_run[0] = m_run[1] = -INFINITY;
            l_run[0] = l_run[1] = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
        }

        const uint32_t sbase = ring + stage * DEC_STAGE_BYTES;
        float s[2][4];
        int nv[2];
#pragma unroll
        for (int pi = 0; pi < 2; ++pi) {
            const int pg = warp * 2 + pi;
            nv[pi] = max(0, min(BN_PAGE_TOKENS, mt.ntok - pg * BN_PAGE_TOKENS));
            if (p.debug & 1) nv[pi] = 0;
            const uint32_t box = sbase + pg * DEC_BOX_BYTES;
#pragma unroll
            for (int j = 0; j < 4; ++j) s[pi][j] = 0.f;
            if (nv[pi] == 0) continue;
            if (nv[pi] < BN_PAGE_TOKENS) {
                // ragged last page: the unwritten V rows may hold anything; 0 * NaN must not reach O
                for (int e = lane; e < (BN_PAGE_TOKENS - nv[pi]) * 8; e += 32) {
                    int row = BN_PAGE_TOKENS + nv[pi] + e / 8;
                    asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(box + row * 128 + (e % 8) * 16), "r"(0)
                                 : "memory");
                }
                __syncwarp();
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const int mat = lane / 8, tok = (lane % 8) + (mat & 1) * 8, chunk16 = kk * 2 + (mat >> 1);
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4(box + tok * 128 + ((chunk16 ^ (tok & 7)) << 4), a0, a1, a2, a3);
                mma_bf16_16816(s[pi], a0, a1, a2, a3, qb[kk][0], qb[kk][1]);
            }
        }
        // online softmax, base 2; thread owns heads hA, hA+1 and tokens lane/4 (+8) of each page
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int pi = 0; pi < 2; ++pi)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int tok = lane / 4 + (j >> 1) * 8;
                s[pi][j] = tok < nv[pi] ? s[pi][j] * p.scale_log2 : -INFINITY;
                tmax[j & 1] = fmaxf(tmax[j & 1], s[pi][j]);
            }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 4));
            tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 8));
            tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 16));
        }
        float msafe[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const float m_new = fmaxf(m_run[hh], tmax[hh]);
            msafe[hh] = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = ex2(m_run[hh] - msafe[hh]);
            m_run[hh] = m_new;
            l_run[hh] *= alpha;
#pragma unroll
            for (int i = 0; i < 4; ++i) { o[i][hh] *= alpha; o[i][hh + 2] *= alpha; }
        }
#pragma unroll
        for (int pi = 0; pi < 2; ++pi) {
            if (nv[pi] == 0) continue;
            float pr[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                pr[j] = ex2(s[pi][j] - msafe[j & 1]);
                l_run[j & 1] += pr[j];
            }
            const uint32_t b0 = movmatrix_trans(pack_bf16(pr[0], pr[1]));
            const uint32_t b1 = movmatrix_trans(pack_bf16(pr[2], pr[3]));
            const uint32_t vbox = sbase + (warp * 2 + pi) * DEC_BOX_BYTES + BN_PAGE_TOKENS * 128;
#pragma unroll
            for (int mtile = 0; mtile < 4; ++mtile) {
                const int mat = lane / 8, tok = (lane % 8) + (mat >> 1) * 8, chunk16 = mtile * 2 + (mat & 1);
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4_trans(vbox + tok * 128 + ((chunk16 ^ (tok & 7)) << 4), a0, a1, a2, a3);
                mma_bf16_16816(o[mtile], a0, a1, a2, a3, b0, b1);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&empty_bar[stage]));
        if (++stage == DEC_NSTAGES) { stage = 0; phase ^= 1u; }

        if (!mt.last) continue;
#if (BN_DDBG & 4)
        continue;
#endif

        // ------------------------------------------------ merge the 4 warps
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 4);
            l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 8);
            l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 16);
        }
        if (lane < 4) {
            mrg_m[warp][hA] = m_run[0]; mrg_m[warp][hA + 1] = m_run[1];
            mrg_l[warp][hA] = l_run[0]; mrg_l[warp][hA + 1] = l_run[1];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int d = i * 16 + lane / 4;
            mrg_o[warp][hA][d] = o[i][0];
            mrg_o[warp][hA + 1][d] = o[i][1];
            mrg_o[warp][hA][d + 8] = o[i][2];
            mrg_o[warp][hA + 1][d + 8] = o[i][3];
        }
        if (!group_sync()) break;
        // thread -> head th, dims td..td+3
        const int th = tid / 16, td = (tid % 16) * 4;
        float mstar = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_CWARPS; ++w) mstar = fmaxf(mstar, mrg_m[w][th]);
        const float ms = mstar == -INFINITY ? 0.f : mstar;
        float lsum = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int w = 0; w < DEC_CWARPS; ++w) {
            const float sc = ex2(mrg_m[w][th] - ms);
            lsum += mrg_l[w][th] * sc;
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] += mrg_o[w][th][td + j] * sc;
        }
        const int bgi = b * p.Hkv + g;
        bool write_final = mt.n_chunks == 1;
        if (!write_final) {
            const size_t slot = (size_t)bgi * p.max_chunks + mt.chunk;
            if (tid % 16 == 0) {
                p.part_m[slot * DEC_G + th] = mstar;
                p.part_l[slot * DEC_G + th] = lsum;
            }
            *reinterpret_cast<float4*>(p.part_o + (slot * DEC_G + th) * DEC_D + td) =
                make_float4(acc[0], acc[1], acc[2], acc[3]);
            __threadfence();
            if (!group_sync()) break;
            if (tid == 0) s_ticket = atomicAdd(&p.tickets[bgi], 1);
            if (!group_sync()) break;
            if (s_ticket == mt.n_chunks - 1) {
                // this CTA finished the last chunk of (b, g): log-sum-exp combine of all partials
                __threadfence();
                const size_t base = (size_t)bgi * p.max_chunks;
                mstar = -INFINITY;
                for (int c = 0; c < mt.n_chunks; ++c) mstar = fmaxf(mstar, __ldcg(p.part_m + (base + c) * DEC_G + th));
                const float ms2 = mstar == -INFINITY ? 0.f : mstar;
                lsum = 0.f;
                acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                for (int c = 0; c < mt.n_chunks; ++c) {
                    const float sc = ex2(__ldcg(p.part_m + (base + c) * DEC_G + th) - ms2);
                    lsum += __ldcg(p.part_l + (base + c) * DEC_G + th) * sc;
                    const float4 po = __ldcg(reinterpret_cast<const float4*>(p.part_o + ((base + c) * DEC_G + th) * DEC_D + td));
                    acc[0] += po.x * sc; acc[1] += po.y * sc; acc[2] += po.z * sc; acc[3] += po.w * sc;
                }
                if (tid == 0) p.tickets[bgi] = 0;   // leave the scratch clean for the next launch
                write_final = true;
            }
        }
        if (write_final && th < p.n_rep) {
            const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
            const size_t row = (size_t)b * p.Hq + (size_t)g * p.n_rep + th;
            const float r0 = acc[0] * inv, r1 = acc[1] * inv, r2 = acc[2] * inv, r3 = acc[3] * inv;
            if (p.out) {
                uint2 v = make_uint2(pack_bf16(r0, r1), pack_bf16(r2, r3));
                *reinterpret_cast<uint2*>(p.out + row * DEC_D + td) = v;
            }
            if (p.out_f32) *reinterpret_cast<float4*>(p.out_f32 + row * DEC_D + td) = make_float4(r0, r1, r2, r3);
            if (p.lse && tid % 16 == 0) p.lse[row] = lsum > 0.f ? (mstar + log2f(lsum)) * LN2 : -INFINITY;
        }
        if (!group_sync()) break;   // mrg_* may be overwritten by the next item after this point
    }
    if (s_abort && lane == 0) atomicExch(&p.hdr->error, BN_ERR_TIMEOUT);
}

// ---------------------------------------------------------------------------
// LSE combine of P partial results (used for the cross-GPU sequence split)
// ---------------------------------------------------------------------------
__global__ void lse_combine_kernel(const float* __restrict__ outs, const float* __restrict__ lses, int P, int64_t n,
                                   int D, float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_bf16,
                                   float* __restrict__ lse) {
    const int64_t row = blockIdx.x;
    float mstar = -INFINITY;
    for (int pp = 0; pp < P; ++pp) mstar = fmaxf(mstar, lses[(int64_t)pp * n + row]);
    const float ms = mstar == -INFINITY ? 0.f : mstar;
    float tot = 0.f;
    for (int pp = 0; pp < P; ++pp) tot += expf(lses[(int64_t)pp * n + row] - ms);
    const float inv = tot > 0.f ? 1.f / tot : 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.f;
        for (int pp = 0; pp < P; ++pp) {
            const float l = lses[(int64_t)pp * n + row];
            if (l > -INFINITY) acc += outs[((int64_t)pp * n + row) * D + d] * expf(l - ms);
        }
        acc *= inv;
        if (out_f32) out_f32[row * D + d] = acc;
        if (out_bf16) out_bf16[row * D + d] = __float2bfloat16(acc);
    }
    if (lse && threadIdx.x == 0) lse[row] = tot > 0.f ? ms + logf(tot) : -INFINITY;
}

}  // namespace bn

using namespace bn;

extern "C" size_t bn_attn_decode_workspace_bytes(int B, int Hq, int Hkv, int D, int max_seq_len, int chunk_tokens) {
    (void)Hq;
    if (B <= 0 || Hkv <= 0 || D != DEC_D || max_seq_len < 0) return 0;
    if (chunk_tokens < 0 || chunk_tokens % DEC_STAGE_TOKENS) return 0;
    int chunk = pick_chunk(B, Hkv, max_seq_len, chunk_tokens);
    return decode_layout(B, Hkv, max_seq_len, chunk).total;
}

extern "C" int bn_attn_decode_paged(const void* q, const void* pool, int64_t pool_pages, const int32_t* page_table,
                                    int max_pages, const int32_t* seq_lens, const int32_t* q_positions, void* out,
                                    float* out_f32, float* lse, int B, int Hq, int Hkv, int D, float scale,
                                    float theta, int rope_q, int max_seq_len, int chunk_tokens, void* workspace,
                                    size_t workspace_bytes, bn_stream_t stream) {
    if (!q || !pool || !page_table || !seq_lens) return fail(BN_ERR_INVALID_ARG, "bn_attn_decode_paged: null pointer");
    if (!out && !out_f32) return fail(BN_ERR_INVALID_ARG, "bn_attn_decode_paged: no output buffer");
    if (B < 0 || Hq <= 0 || Hkv <= 0 || max_pages < 0 || max_seq_len < 0 || pool_pages <= 0)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_decode_paged: bad sizes B=%d Hq=%d Hkv=%d max_pages=%d", B, Hq, Hkv,
                    max_pages);
    if (D != DEC_D) return fail(BN_ERR_UNSUPPORTED, "bn_attn_decode_paged: head_dim=%d (64 supported)", D);
    if (Hq % Hkv != 0 || Hq / Hkv > DEC_G)
        return fail(BN_ERR_UNSUPPORTED, "bn_attn_decode_paged: Hq/Hkv=%d/%d (group of 1..8 supported)", Hq, Hkv);
    if (chunk_tokens < 0 || chunk_tokens % DEC_STAGE_TOKENS)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_decode_paged: chunk_tokens=%d must be 0 or a multiple of %d",
                    chunk_tokens, DEC_STAGE_TOKENS);
    if ((int64_t)max_pages * BN_PAGE_TOKENS < max_seq_len)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_decode_paged: max_pages=%d cannot hold max_seq_len=%d", max_pages,
                    max_seq_len);
    if (pool_pages * Hkv * DEC_BOX_ROWS > 0x7fffffffLL)
        return fail(BN_ERR_UNSUPPORTED, "bn_attn_decode_paged: pool of %lld pages is too large", (long long)pool_pages);
    if ((reinterpret_cast<uintptr_t>(q) & 3) || (out && (reinterpret_cast<uintptr_t>(out) & 7)) ||
        (out_f32 && (reinterpret_cast<uintptr_t>(out_f32) & 15)))
        return fail(BN_ERR_INVALID_ARG, "bn_attn_decode_paged: q/out buffers must be 4/8/16-byte aligned");
    if (int rc = require_sm100()) return rc;
    if (B == 0) return BN_OK;
    const int chunk = pick_chunk(B, Hkv, max_seq_len, chunk_tokens);
    const DecodeLayout L = decode_layout(B, Hkv, max_seq_len, chunk);
    if (!workspace || workspace_bytes < L.total)
        return fail(BN_ERR_WORKSPACE, "bn_attn_decode_paged: workspace of %zu bytes given, %zu needed", workspace_bytes,
                    L.total);
    if (reinterpret_cast<uintptr_t>(workspace) & 255)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_decode_paged: workspace must be 256-byte aligned");

    CUtensorMap tmap;
    const uint64_t dims[2] = {(uint64_t)DEC_D, (uint64_t)pool_pages * Hkv * DEC_BOX_ROWS};
    const uint64_t strides[1] = {DEC_D * 2};
    const uint32_t box[2] = {DEC_D, DEC_BOX_ROWS};
    if (int rc = make_tensor_map(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, pool, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
        return rc;

    uint8_t* ws = static_cast<uint8_t*>(workspace);
    DecodeParams p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.page_table = page_table;
    p.seq_lens = seq_lens;
    p.q_positions = q_positions;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.out_f32 = out_f32;
    p.lse = lse;
    p.hdr = reinterpret_cast<DecodeHeader*>(ws);
    p.tickets = reinterpret_cast<int*>(ws + L.tickets);
    p.part_m = reinterpret_cast<float*>(ws + L.part_m);
    p.part_l = reinterpret_cast<float*>(ws + L.part_l);
    p.part_o = reinterpret_cast<float*>(ws + L.part_o);
    p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.n_rep = Hq / Hkv; p.max_pages = max_pages; p.max_seq_len = max_seq_len;
    p.chunk = chunk; p.max_chunks = L.max_chunks;
    p.total_items = B * Hkv * L.max_chunks;
    p.rope_q = rope_q;
    { const char* e = getenv("BN_DECODE_DEBUG"); p.debug = e ? atoi(e) : 0; }
    p.scale_log2 = scale * LOG2E;
    p.theta = theta;

    static thread_local int configured_dev = -1;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(decode_paged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             DEC_SMEM_BYTES);
        if (e != cudaSuccess) return fail(BN_ERR_CUDA, "cudaFuncSetAttribute(decode): %s", cudaGetErrorString(e));
        configured_dev = dev;
    }
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int grid = p.total_items < sms ? p.total_items : sms;
    decode_paged_kernel<<<grid, DEC_THREADS, DEC_SMEM_BYTES, as_stream(stream)>>>(tmap, p);
    return launch_status("bn_attn_decode_paged");
}

extern "C" int bn_attn_lse_combine(const float* outs, const float* lses, int P, int64_t n, int D, float* out_f32,
                                   void* out_bf16, float* lse, bn_stream_t stream) {
    if (!outs || !lses || (!out_f32 && !out_bf16)) return fail(BN_ERR_INVALID_ARG, "bn_attn_lse_combine: null pointer");
    if (P <= 0 || n < 0 || D <= 0) return fail(BN_ERR_INVALID_ARG, "bn_attn_lse_combine: bad sizes P=%d D=%d", P, D);
    if (int rc = require_sm100()) return rc;
    if (n == 0) return BN_OK;
    lse_combine_kernel<<<(unsigned)n, 64, 0, as_stream(stream)>>>(outs, lses, P, n, D, out_f32,
                                                                static_cast<__nv_bfloat16*>(out_bf16), lse);
    return launch_status("bn_attn_lse_combine");
}

// Single-token decode attention over the paged bf16 KV cache (HBM-bound).
//
// Decode semantics follow the reference's generate loop, where the new token's
// output is the last row of an attention over everything before it
// (mygrad/llama/llama_model.py:136-144); here the earlier keys/values come from
// the cache instead of being recomputed.
//
// Design (one persistent CTA per SM, no scheduling atomics):
//   * The work of the launch is the sequence of all 128-token stages, ordered by
//     (sequence, KV head, position).  It is cut into equal contiguous ranges,
//     one per CTA, so every SM streams the same number of bytes whatever the
//     sequence lengths are.  A range is a list of segments = (sequence, KV head,
//     run of stages); every warp derives the list from seq_lens by itself.
//   * A producer warp streams the pages of its range through a ring of
//     shared-memory stages with TMA tensor loads (one 4 KB box = K and V of one
//     (page, head), 128-byte swizzle), completion counted on mbarriers; page
//     numbers are fetched one stage ahead.
//   * Eight consumer warps each take two pages (32 tokens) of a stage, as two
//     independent instruction chains.  All 8
//     query heads of the GQA group are served from the one K/V read:
//       S^T (16 tokens x 8 heads) = K_page (16 x 64) . Q^T (64 x 8)
//       O^T (64 dims  x 8 heads) += V_page^T (64 x 16) . P^T (16 x 8)
//     as m16n8k16 bf16 MMAs with fp32 accumulation; softmax is online, base 2.
//   * At the end of a segment the consumer warps merge (m, l, O) in shared
//     memory.  A (sequence, head) that spans several CTAs leaves fp32 partials
//     in scratch memory; a tenth warp takes the ticket for it and, in the CTA
//     that delivers the last partial, performs the log-sum-exp combine (nobody
//     spins on another CTA) and re-arms the ticket, so that the consumers never
//     wait on global memory at a segment boundary.
//   * Every wait is bounded; on expiry the kernel raises the error word in the
//     scratch header and returns.
#include <math.h>

#include "common.cuh"
#include "ptx.cuh"
#include "tma.cuh"

namespace bn {

using namespace ptx;

constexpr int DEC_D = 64;
constexpr int DEC_G = 8;                    // query heads per KV head served by one MMA (n = 8)
constexpr int DEC_STAGE_TOKENS = 256;
constexpr int DEC_PAGES_PER_STAGE = DEC_STAGE_TOKENS / BN_PAGE_TOKENS;  // 16
constexpr int DEC_BOX_ROWS = 2 * BN_PAGE_TOKENS;                        // K rows then V rows
constexpr int DEC_BOX_BYTES = DEC_BOX_ROWS * DEC_D * 2;                 // 4096
constexpr int DEC_STAGE_BYTES = DEC_PAGES_PER_STAGE * DEC_BOX_BYTES;    // 65536
constexpr int DEC_NSTAGES = 3;
constexpr int DEC_CWARPS = 8;                                            // consumer warps
constexpr int DEC_PPW = DEC_PAGES_PER_STAGE / DEC_CWARPS;                // pages per warp and stage
constexpr int DEC_CTHREADS = DEC_CWARPS * 32;
constexpr int DEC_DPT = DEC_G * DEC_D / DEC_CTHREADS;                    // output dims per thread in the merge (2)
constexpr int DEC_TPH = DEC_D / DEC_DPT;                                 // threads per head in the merge
constexpr int DEC_THREADS = (DEC_CWARPS + 2) * 32;                      // + producer warp + combine warp
constexpr int DEC_SMEM_BYTES = DEC_NSTAGES * DEC_STAGE_BYTES + 1024;
constexpr int DEC_MAX_SEQS = 1024;          // sequences per launch (prefix table in shared memory)
constexpr int DEC_DEFAULT_MIN_TOKENS = 1024;   // a CTA's range is never shorter than this
constexpr int DEC_WHOLE_MAX_STAGES = 8;        // sequences up to this many stages are never split (if there are enough of them)
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct DecodeHeader {   // first 256 bytes of the scratch buffer
    int error;          // BN_ERR_TIMEOUT once a bounded wait ran out
};

struct DecodeLayout {
    size_t tickets, part_m, part_l, part_o, total;
    int max_parts;      // partial slots per (sequence, KV head)
};

// `ticket_slots` is the capacity of the ticket region, NOT B * Hkv: the tickets are the only words of the scratch
// that outlive a launch (a merging CTA re-arms the ones it used), so their place must not move with the batch
// size, or a later, larger batch would find its tickets where an earlier call wrote partials.
static DecodeLayout decode_layout(int B, int Hkv, int max_seq_len, int min_tokens, size_t ticket_slots) {
    DecodeLayout L;
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    // a (sequence, head) of n stages overlaps at most n / (min stages per CTA) + 2 CTA ranges
    L.max_parts = (max_seq_len + min_tokens - 1) / min_tokens + 2;
    size_t bg = (size_t)B * Hkv;
    L.tickets = 256;
    L.part_m = L.tickets + up(ticket_slots * sizeof(int));
    L.part_l = L.part_m + up(bg * L.max_parts * DEC_G * sizeof(float));
    L.part_o = L.part_l + up(bg * L.max_parts * DEC_G * sizeof(float));
    L.total = L.part_o + up(bg * L.max_parts * DEC_G * DEC_D * sizeof(float));
    return L;
}

// caller-owned scratch: room for the tickets of the largest batch a launch accepts, whatever B this call has
static size_t regular_ticket_slots(int Hkv) { return (size_t)DEC_MAX_SEQS * Hkv; }

static int pick_min_tokens(int chunk_tokens) {
    const int t = chunk_tokens > 0 ? chunk_tokens : DEC_DEFAULT_MIN_TOKENS;
    return (t + DEC_STAGE_TOKENS - 1) / DEC_STAGE_TOKENS * DEC_STAGE_TOKENS;   // whole stages
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
    int B, Hq, Hkv, n_rep, max_pages, max_seq_len, min_stages, max_parts, rope_q;
    float scale_log2, theta;
};

// The launch-wide schedule, derived from seq_lens by every thread of every CTA.
struct Schedule {
    const int* prefix;     // shared memory: prefix[b] = sum of stages of sequences < b (one KV head)
    const int* len;        // shared memory: clamped sequence lengths
    int Hkv, B;
    int T;                 // all stages of the launch (< 2^31)
    int G;                 // CTAs that take part
    bool whole;            // short sequences: a CTA takes whole (sequence, KV head) segments, nothing is split
    __device__ __forceinline__ int nst(int b) const { return prefix[b + 1] - prefix[b]; }
    // 32-bit division whenever the products fit (G <= 2^9 CTAs, T < 2^22 stages): the 64-bit form is an emulated
    // sequence several times longer, and these sit on the path to the first TMA load
    __device__ __forceinline__ bool small() const { return T < (1 << 22) && G <= (1 << 9); }
    __device__ __forceinline__ int range_begin(int cta) const {
        if (whole) {
            // segments [cta * n / G, (cta + 1) * n / G) of the n = B * Hkv segments, in (sequence, head) order
            const int n = B * Hkv, k = (int)((unsigned)cta * (unsigned)n / (unsigned)G);
            if (k >= n) return T;
            const int b = k / Hkv;
            return Hkv * prefix[b] + (k - b * Hkv) * nst(b);
        }
        return small() ? (int)((unsigned)cta * (unsigned)T / (unsigned)G) : (int)((long long)cta * T / G);
    }
    // the CTA whose range holds global stage x
    __device__ __forceinline__ int cta_of(int x) const {
        return small() ? (int)((((unsigned)x + 1u) * (unsigned)G - 1u) / (unsigned)T)
                       : (int)((((long long)x + 1) * G - 1) / T);
    }
    // first sequence b with Hkv * prefix[b + 1] > x
    __device__ __forceinline__ int seq_of(int x) const {
        int lo = 0, hi = B - 1;
        while (lo < hi) {
            int mid = (lo + hi) >> 1;
            if (Hkv * prefix[mid + 1] > x) hi = mid; else lo = mid + 1;
        }
        return lo;
    }
};

// One segment of a CTA's range: stages [s0, s1) of (b, g).
struct Segment {
    int b, g, s0, s1, L;
    int c_first, n_parts;   // CTAs that hold a piece of this (b, g)
};

// Walks the segments of the range [pos, end).  Only the first step searches; later ones step to the next
// KV head / sequence.  Division-heavy lookups happen only for the (at most two) segments that a range
// boundary cuts.
struct SegmentIter {
    int pos, end, b, g;
    bool started;
    __device__ __forceinline__ void init(int lo, int hi) { pos = lo; end = hi; b = 0; g = 0; started = false; }
    // `want_parts` = false skips c_first / n_parts (two divisions), which the producer never reads
    __device__ __forceinline__ bool next(const Schedule& sc, Segment& sg, bool want_parts = true) {
        if (pos >= end) return false;
        int n;
        if (!started) {
            b = sc.seq_of(pos);
            n = sc.nst(b);
            g = (pos - sc.Hkv * sc.prefix[b]) / n;
            started = true;
        } else {
            if (++g == sc.Hkv) {
                g = 0;
                do { ++b; } while (sc.nst(b) == 0);
            }
            n = sc.nst(b);
        }
        const int sb = sc.Hkv * sc.prefix[b] + g * n;
        sg.b = b; sg.g = g;
        sg.s0 = pos - sb;
        sg.s1 = min(n, end - sb);
        sg.L = sc.len[b];
        if ((sg.s0 == 0 && sg.s1 == n) || !want_parts) {
            sg.c_first = blockIdx.x;
            sg.n_parts = 1;
        } else {
            sg.c_first = sc.cta_of(sb);
            sg.n_parts = sc.cta_of(sb + n - 1) - sg.c_first + 1;
        }
        pos = sb + sg.s1;
        return true;
    }
};

__global__ void __launch_bounds__(DEC_THREADS, 1)
decode_paged_kernel(const __grid_constant__ CUtensorMap tmap, const DecodeParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[DEC_NSTAGES];
    __shared__ __align__(8) uint64_t empty_bar[DEC_NSTAGES];
    __shared__ __align__(8) uint64_t merge_bar, part_bar;
    __shared__ int s_prefix[DEC_MAX_SEQS + 1];
    __shared__ int s_len[DEC_MAX_SEQS];
    __shared__ int s_nmax;                      // stages of the longest sequence
    __shared__ float mrg_m[DEC_CWARPS][DEC_G], mrg_l[DEC_CWARPS][DEC_G];
    __shared__ __align__(16) float mrg_o[DEC_CWARPS][DEC_G][DEC_D + 2];   // read back as float2
    __shared__ __align__(16) __nv_bfloat16 s_q[DEC_G][DEC_D];   // rotated query heads of the current segment
    __shared__ float s_inv_freq[DEC_D / 2];
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;

    if (tid == 0) {
        for (int s = 0; s < DEC_NSTAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), DEC_CWARPS);
        }
        mbar_init(smem_u32(&merge_bar), DEC_CWARPS);
        mbar_init(smem_u32(&part_bar), DEC_CWARPS);
        s_abort = 0;
        fence_mbar_init();
        prefetch_tensormap(&tmap);
    }
    // Everything above touches no global memory, so with a programmatic dependent launch it overlaps the tail of
    // the previous kernel of the stream; nothing below runs before that kernel's writes are visible.
    grid_dependency_wait();
    grid_launch_dependents();
    // stages per sequence, then an exclusive prefix sum (warp 0)
    for (int b = tid; b < p.B; b += DEC_THREADS) {
        const int L = max(0, min(p.seq_lens[b], p.max_seq_len));
        s_len[b] = L;
        s_prefix[b + 1] = (L + DEC_STAGE_TOKENS - 1) / DEC_STAGE_TOKENS;
    }
    __syncthreads();
    if (warp == 0) {
        int carry = 0, nmax = 0;
        for (int b0 = 0; b0 < p.B; b0 += 32) {
            const int b = b0 + lane;
            int v = b < p.B ? s_prefix[b + 1] : 0;
            nmax = max(nmax, v);
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += t;
            }
            if (b < p.B) s_prefix[b + 1] = carry + v;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
        nmax = __reduce_max_sync(0xffffffffu, nmax);
        if (lane == 0) { s_prefix[0] = 0; s_nmax = nmax; }
    }
    __syncthreads();

    Schedule sc;
    sc.prefix = s_prefix;
    sc.len = s_len;
    sc.Hkv = p.Hkv;
    sc.B = p.B;
    sc.T = p.Hkv * s_prefix[p.B];
    // Equal shares of the stage stream cut segments wherever a share ends, and every cut costs a partial result, a
    // ticket and a merge.  That is the right trade for long sequences; when no sequence is longer than 8 stages (2048
    // tokens) and there are at least 16 segments, a cut costs more than the imbalance it removes (16 sequences of 576
    // tokens: 7.1 us with whole segments against 9.3 - 10.9 us with equal shares), so CTAs take whole segments.
    sc.whole = s_nmax <= DEC_WHOLE_MAX_STAGES && p.B * p.Hkv >= 16;
    sc.G = sc.whole ? min((int)gridDim.x, p.B * p.Hkv) : max(1, min((int)gridDim.x, sc.T / p.min_stages));
    const bool active = sc.T > 0 && (int)blockIdx.x < sc.G;
    const int range_lo = active ? sc.range_begin(blockIdx.x) : 0;
    const int range_hi = active ? sc.range_begin(blockIdx.x + 1) : 0;

    if (warp == DEC_CWARPS) {
        // ------------------------------------------------------------ producer
        // Page numbers are read a group of 4 stages (32 pages, one 128-byte line of the page table) at a
        // time, one group ahead of their use and across segment boundaries, so that the TMA issue never
        // waits on a page-table load.
        constexpr int GRP = 32 / DEC_PAGES_PER_STAGE;   // stages per group
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        SegmentIter iter;
        iter.init(range_lo, range_hi);
        Segment sg, sg_next;
        bool have = iter.next(sc, sg, false);
        auto load_group = [&](const Segment& sgm, int grp) {
            const int e = grp * 32 + lane;
            const int n_pages_seq = (sgm.L + BN_PAGE_TOKENS - 1) / BN_PAGE_TOKENS;
            return e < n_pages_seq ? p.page_table[(size_t)sgm.b * p.max_pages + e] : -1;
        };
        const uint64_t stream_policy = l2_policy_evict_first();     // every cache byte is read once per launch
        int ids = have ? load_group(sg, sg.s0 / GRP) : -1, ids_pref = -1;
        while (ok && have) {
            const bool have_next = iter.next(sc, sg_next, false);
            const int n_pages_seq = (sg.L + BN_PAGE_TOKENS - 1) / BN_PAGE_TOKENS;
            for (int s = sg.s0; s < sg.s1; ++s) {
                if (s == sg.s0 || s % GRP == 0) {
                    if (s != sg.s0) ids = ids_pref;
                    const int grp = s / GRP;
                    if ((grp + 1) * GRP < sg.s1) ids_pref = load_group(sg, grp + 1);
                    else if (have_next) ids_pref = load_group(sg_next, sg_next.s0 / GRP);
                }
                const int page = __shfl_sync(0xffffffffu, ids, (s % GRP) * DEC_PAGES_PER_STAGE + (lane % DEC_PAGES_PER_STAGE));
                if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, &s_abort)) { ok = false; break; }
                const int npages = min(DEC_PAGES_PER_STAGE, n_pages_seq - s * DEC_PAGES_PER_STAGE);
                const uint32_t fb = smem_u32(&full_bar[stage]);
                if (lane == 0) mbar_arrive_expect_tx(fb, (uint32_t)npages * DEC_BOX_BYTES);
                __syncwarp();
                if (lane < npages && page >= 0)
                    tma_load_2d_hint(ring + stage * DEC_STAGE_BYTES + lane * DEC_BOX_BYTES, &tmap, 0,
                                     (page * p.Hkv + sg.g) * DEC_BOX_ROWS, fb, stream_policy);
                if (++stage == DEC_NSTAGES) { stage = 0; phase ^= 1u; }
            }
            sg = sg_next;
            ids = ids_pref;
            have = have_next;
        }
        if (lane == 0 && s_abort) atomicExch(&p.hdr->error, BN_ERR_TIMEOUT);
        return;
    }

    if (warp == DEC_CWARPS + 1) {
        // -------------------------------------------------------- combine warp
        // For every segment of this CTA that is only a part of its (sequence, head): wait until the consumers
        // have stored the partial, take a ticket, and in the CTA that holds the last ticket merge all parts.
        SegmentIter iter;
        iter.init(range_lo, range_hi);
        Segment sg;
        uint32_t pphase = 0;
        while (iter.next(sc, sg)) {
            if (sg.n_parts == 1) continue;
            if (!mbar_wait(smem_u32(&part_bar), pphase, &s_abort)) break;
            pphase ^= 1u;
            __threadfence();     // the consumers' stores, observed through the barrier, before the ticket
            const int bgi = sg.b * p.Hkv + sg.g;
            int ticket = 0;
            if (lane == 0) ticket = atomicAdd(&p.tickets[bgi], 1);
            ticket = __shfl_sync(0xffffffffu, ticket, 0);
            if (ticket != sg.n_parts - 1) continue;
            __threadfence();
            const size_t base = (size_t)bgi * p.max_parts;
            // lane -> head lane / 4, dims 16 * (lane % 4) .. + 15
            const int ch = lane / 4, cd = (lane % 4) * 16;
            // parts are merged four at a time: all their loads are issued before the first use, so a merge of up
            // to four parts costs one L2 round trip, not one per part
            float m2 = -INFINITY, l2 = 0.f, a2[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) a2[i] = 0.f;
            for (int c0 = 0; c0 < sg.n_parts; c0 += 4) {
                float pm[4], pl[4];
                float4 po[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const bool on = c0 + i < sg.n_parts;
                    const size_t e = (base + (on ? c0 + i : 0)) * DEC_G + ch;
                    pm[i] = on ? __ldcg(p.part_m + e) : -INFINITY;
                    pl[i] = on ? __ldcg(p.part_l + e) : 0.f;
                    const float4* src = reinterpret_cast<const float4*>(p.part_o + e * DEC_D + cd);
#pragma unroll
                    for (int v = 0; v < 4; ++v) po[i][v] = on ? __ldcg(src + v) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                float mnew = m2;
#pragma unroll
                for (int i = 0; i < 4; ++i) mnew = fmaxf(mnew, pm[i]);
                const float ms2 = mnew == -INFINITY ? 0.f : mnew;
                const float keep = ex2(m2 - ms2);          // 0 while nothing has been merged yet (m2 = -inf)
                l2 *= keep;
#pragma unroll
                for (int i = 0; i < 16; ++i) a2[i] *= keep;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float scl = ex2(pm[i] - ms2);
                    l2 += pl[i] * scl;
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        a2[4 * v] += po[i][v].x * scl; a2[4 * v + 1] += po[i][v].y * scl;
                        a2[4 * v + 2] += po[i][v].z * scl; a2[4 * v + 3] += po[i][v].w * scl;
                    }
                }
                m2 = mnew;
            }
            if (lane == 0) p.tickets[bgi] = 0;   // leave the scratch clean for the next launch
            if (ch < p.n_rep) {
                const float inv = l2 > 0.f ? 1.f / l2 : 0.f;
                const size_t crow = (size_t)sg.b * p.Hq + (size_t)sg.g * p.n_rep + ch;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float r0 = a2[4 * i] * inv, r1 = a2[4 * i + 1] * inv, r2 = a2[4 * i + 2] * inv,
                                r3 = a2[4 * i + 3] * inv;
                    if (p.out)
                        *reinterpret_cast<uint2*>(p.out + crow * DEC_D + cd + 4 * i) =
                            make_uint2(pack_bf16(r0, r1), pack_bf16(r2, r3));
                    if (p.out_f32)
                        *reinterpret_cast<float4*>(p.out_f32 + crow * DEC_D + cd + 4 * i) = make_float4(r0, r1, r2, r3);
                }
                if (p.lse && lane % 4 == 0) p.lse[crow] = l2 > 0.f ? (m2 + log2f(l2)) * LN2 : -INFINITY;
            }
        }
        if (lane == 0 && s_abort) atomicExch(&p.hdr->error, BN_ERR_TIMEOUT);
        return;
    }

    // --------------------------------------------------------------- consumers
    // sequences without tokens get a zero output from whoever passes by
    for (int bgi = blockIdx.x; bgi < p.B * p.Hkv; bgi += gridDim.x) {
        const int b = bgi / p.Hkv, g = bgi % p.Hkv;
        if (sc.nst(b) > 0) continue;
        const int th = tid / DEC_TPH, td = (tid % DEC_TPH) * DEC_DPT;
        if (th >= p.n_rep) continue;
        const size_t row = (size_t)b * p.Hq + (size_t)g * p.n_rep + th;
        if (p.out) *reinterpret_cast<uint32_t*>(p.out + row * DEC_D + td) = 0u;
        if (p.out_f32) *reinterpret_cast<float2*>(p.out_f32 + row * DEC_D + td) = make_float2(0.f, 0.f);
        if (p.lse && tid % DEC_TPH == 0) p.lse[row] = -INFINITY;
    }

    int stage = 0;
    uint32_t phase = 0, mphase = 0;
    const int hA = 2 * (lane % 4);       // the two heads whose softmax state this thread carries
    const uint32_t mb = smem_u32(&merge_bar);
    auto group_sync = [&]() -> bool {
        __syncwarp();
        if (lane == 0) mbar_arrive(mb);
        const bool ok = mbar_wait(mb, mphase, &s_abort);
        mphase ^= 1u;
        return ok;
    };
    // raw query pair of thread (head tid / 32, dims 2 * (tid % 32), + 1) for a segment
    auto load_q_raw = [&](const Segment& sg) -> uint32_t {
        const int th = tid / DEC_TPH, td = (tid % DEC_TPH) * DEC_DPT;
        if (th >= p.n_rep) return 0u;
        return *reinterpret_cast<const uint32_t*>(p.q + ((size_t)sg.b * p.Hq + (size_t)sg.g * p.n_rep + th) * DEC_D + td);
    };

    // rotate the 8 query heads of a segment (one pair per thread) into shared memory
    auto store_q = [&](const Segment& sgq, uint32_t raw) {
        const int th = tid / DEC_TPH, td = (tid % DEC_TPH) * DEC_DPT;
        const int qpos = p.q_positions ? p.q_positions[sgq.b] : sgq.L - 1;
        float x0 = bf16_lo(raw), x1 = bf16_hi(raw);
        if (p.rope_q) {
            const float angle = qpos * s_inv_freq[td / 2];
            float sin_angle, cos_angle;
            sincosf(angle, &sin_angle, &cos_angle);
            const float y0 = x0 * cos_angle - x1 * sin_angle;
            const float y1 = x0 * sin_angle + x1 * cos_angle;
            x0 = y0; x1 = y1;
        }
        *reinterpret_cast<uint32_t*>(&s_q[th][td]) = pack_bf16(x0, x1);
    };

    SegmentIter iter;
    iter.init(range_lo, range_hi);
    Segment sg, sg_next;
    bool have = iter.next(sc, sg);
    uint32_t q_raw = have ? load_q_raw(sg) : 0u;
    bool ok = true;
    // the RoPE frequencies are needed by the consumers only; computing them here keeps them off the path to
    // the first TMA load
    if (tid < DEC_D / 2) s_inv_freq[tid] = rope_inv_freq(tid, DEC_D, p.theta);
    ok = group_sync();
    if (ok && have) {
        store_q(sg, q_raw);
        ok = group_sync();
    }
    while (ok && have) {
        // look one segment ahead so that its query is already on the way
        const bool have_next = iter.next(sc, sg_next);
        const uint32_t q_raw_next = have_next ? load_q_raw(sg_next) : 0u;
        // Q^T fragments (k = dims, n = heads)
        uint32_t qb[4][2];
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
#pragma unroll
            for (int h8 = 0; h8 < 2; ++h8)
                qb[kk][h8] = *reinterpret_cast<const uint32_t*>(&s_q[lane / 4][kk * 16 + h8 * 8 + 2 * (lane % 4)]);

        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
        float o[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) o[i][j] = 0.f;

        for (int s = sg.s0; s < sg.s1; ++s) {
            if (!mbar_wait(smem_u32(&full_bar[stage]), phase, &s_abort)) { ok = false; break; }
            const int ntok = min(DEC_STAGE_TOKENS, sg.L - s * DEC_STAGE_TOKENS);
            const uint32_t sbase = ring + stage * DEC_STAGE_BYTES;
            float sv[DEC_PPW][4];
            int nv[DEC_PPW];
#pragma unroll
            for (int pi = 0; pi < DEC_PPW; ++pi) {
                const int pg = warp * DEC_PPW + pi;
                nv[pi] = max(0, min(BN_PAGE_TOKENS, ntok - pg * BN_PAGE_TOKENS));
                const uint32_t box = sbase + pg * DEC_BOX_BYTES;
#pragma unroll
                for (int j = 0; j < 4; ++j) sv[pi][j] = 0.f;
                if (nv[pi] == 0) continue;
                if (nv[pi] < BN_PAGE_TOKENS) {
                    // ragged last page: the unwritten V rows may hold anything; 0 * NaN must not reach O
                    for (int e = lane; e < (BN_PAGE_TOKENS - nv[pi]) * 8; e += 32) {
                        const int row = BN_PAGE_TOKENS + nv[pi] + e / 8;
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
                    mma_bf16_16816(sv[pi], a0, a1, a2, a3, qb[kk][0], qb[kk][1]);
                }
            }
            // online softmax, base 2; thread owns heads hA, hA+1 and tokens lane/4 (+8) of each page
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int pi = 0; pi < DEC_PPW; ++pi)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int tok = lane / 4 + (j >> 1) * 8;
                    sv[pi][j] = tok < nv[pi] ? sv[pi][j] * p.scale_log2 : -INFINITY;
                    tmax[j & 1] = fmaxf(tmax[j & 1], sv[pi][j]);
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
                if (m_new != m_run[hh]) {     // the running maximum moves rarely after the first stages
                    const float alpha = ex2(m_run[hh] - msafe[hh]);
                    m_run[hh] = m_new;
                    l_run[hh] *= alpha;
#pragma unroll
                    for (int i = 0; i < 4; ++i) { o[i][hh] *= alpha; o[i][hh + 2] *= alpha; }
                }
            }
#pragma unroll
            for (int pi = 0; pi < DEC_PPW; ++pi) {
                if (nv[pi] == 0) continue;
                float pr[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    pr[j] = ex2(sv[pi][j] - msafe[j & 1]);
                    l_run[j & 1] += pr[j];
                }
                const uint32_t b0 = movmatrix_trans(pack_bf16(pr[0], pr[1]));
                const uint32_t b1 = movmatrix_trans(pack_bf16(pr[2], pr[3]));
                const uint32_t vbox = sbase + (warp * DEC_PPW + pi) * DEC_BOX_BYTES + BN_PAGE_TOKENS * 128;
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
        }
        if (!ok) break;

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
        // thread -> head th, dims td, td + 1
        const int th = tid / DEC_TPH, td = (tid % DEC_TPH) * DEC_DPT;
        float mstar = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_CWARPS; ++w) mstar = fmaxf(mstar, mrg_m[w][th]);
        const float ms = mstar == -INFINITY ? 0.f : mstar;
        float lsum = 0.f, acc[2] = {0.f, 0.f};
#pragma unroll
        for (int w = 0; w < DEC_CWARPS; ++w) {
            const float scl = ex2(mrg_m[w][th] - ms);
            lsum += mrg_l[w][th] * scl;
            const float2 po = *reinterpret_cast<const float2*>(&mrg_o[w][th][td]);
            acc[0] += po.x * scl; acc[1] += po.y * scl;
        }
        const int bgi = sg.b * p.Hkv + sg.g;
        const size_t row = (size_t)sg.b * p.Hq + (size_t)sg.g * p.n_rep + th;
        auto write_final = [&](float m_, float l_, const float (&a)[2]) {
            if (th >= p.n_rep) return;
            const float inv = l_ > 0.f ? 1.f / l_ : 0.f;
            const float r0 = a[0] * inv, r1 = a[1] * inv;
            if (p.out) *reinterpret_cast<uint32_t*>(p.out + row * DEC_D + td) = pack_bf16(r0, r1);
            if (p.out_f32) *reinterpret_cast<float2*>(p.out_f32 + row * DEC_D + td) = make_float2(r0, r1);
            if (p.lse && tid % DEC_TPH == 0) p.lse[row] = l_ > 0.f ? (m_ + log2f(l_)) * LN2 : -INFINITY;
        };
        if (sg.n_parts == 1) {
            write_final(mstar, lsum, acc);
        } else {
            const size_t slot = (size_t)bgi * p.max_parts + ((int)blockIdx.x - sg.c_first);
            if (tid % DEC_TPH == 0) {
                p.part_m[slot * DEC_G + th] = mstar;
                p.part_l[slot * DEC_G + th] = lsum;
            }
            *reinterpret_cast<float2*>(p.part_o + (slot * DEC_G + th) * DEC_D + td) = make_float2(acc[0], acc[1]);
            // hand the partial to the combine warp and go on
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&part_bar));
        }
        // the next segment's query replaces this one's (every warp took its fragments long ago)
        if (have_next) store_q(sg_next, q_raw_next);
        if (!group_sync()) break;              // mrg_* free again, s_q visible
        sg = sg_next;
        q_raw = q_raw_next;
        have = have_next;
    }
    if (s_abort && lane == 0) atomicExch(&p.hdr->error, BN_ERR_TIMEOUT);
}

// ---------------------------------------------------------------------------
// LSE combine of P partial results (used for the cross-GPU sequence split)
// ---------------------------------------------------------------------------
__global__ void lse_combine_kernel(const float* __restrict__ outs, int64_t outs_part_stride,
                                   const float* __restrict__ lses, int64_t lses_part_stride, int P, int64_t n, int D,
                                   float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_bf16,
                                   float* __restrict__ lse) {
    const int64_t row = blockIdx.x;
    float mstar = -INFINITY;
    for (int pp = 0; pp < P; ++pp) mstar = fmaxf(mstar, lses[pp * lses_part_stride + row]);
    const float ms = mstar == -INFINITY ? 0.f : mstar;
    float tot = 0.f;
    for (int pp = 0; pp < P; ++pp) tot += expf(lses[pp * lses_part_stride + row] - ms);
    const float inv = tot > 0.f ? 1.f / tot : 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.f;
        for (int pp = 0; pp < P; ++pp) {
            const float l = lses[pp * lses_part_stride + row];
            if (l > -INFINITY) acc += outs[pp * outs_part_stride + row * D + d] * expf(l - ms);
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
    if (chunk_tokens < 0 || chunk_tokens % 128) return 0;
    return decode_layout(B, Hkv, max_seq_len, pick_min_tokens(chunk_tokens), regular_ticket_slots(Hkv)).total;
}

static int decode_launch(const void* q, const void* pool, int64_t pool_pages, const int32_t* page_table,
                         int max_pages, const int32_t* seq_lens, const int32_t* q_positions, void* out,
                         float* out_f32, float* lse, int B, int Hq, int Hkv, int D, float scale, float theta,
                         int rope_q, int max_seq_len, int chunk_tokens, void* workspace, size_t workspace_bytes,
                         size_t ticket_slots, bn_stream_t stream) {
    if (!q || !pool || !page_table || !seq_lens) return fail(BN_ERR_INVALID_ARG, "bn_attn_decode_paged: null pointer");
    if (!out && !out_f32) return fail(BN_ERR_INVALID_ARG, "bn_attn_decode_paged: no output buffer");
    if (B < 0 || Hq <= 0 || Hkv <= 0 || max_pages < 0 || max_seq_len < 0 || pool_pages <= 0)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_decode_paged: bad sizes B=%d Hq=%d Hkv=%d max_pages=%d", B, Hq, Hkv,
                    max_pages);
    if (D != DEC_D) return fail(BN_ERR_UNSUPPORTED, "bn_attn_decode_paged: head_dim=%d (64 supported)", D);
    if (Hq % Hkv != 0 || Hq / Hkv > DEC_G)
        return fail(BN_ERR_UNSUPPORTED, "bn_attn_decode_paged: Hq/Hkv=%d/%d (group of 1..8 supported)", Hq, Hkv);
    if (B > DEC_MAX_SEQS)
        return fail(BN_ERR_UNSUPPORTED, "bn_attn_decode_paged: %d sequences in one launch (<= %d supported)", B,
                    DEC_MAX_SEQS);
    if (chunk_tokens < 0 || chunk_tokens % 128)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_decode_paged: chunk_tokens=%d must be 0 or a multiple of 128",
                    chunk_tokens);
    if ((int64_t)max_pages * BN_PAGE_TOKENS < max_seq_len)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_decode_paged: max_pages=%d cannot hold max_seq_len=%d", max_pages,
                    max_seq_len);
    if ((long long)B * Hkv * ((max_seq_len + DEC_STAGE_TOKENS - 1) / DEC_STAGE_TOKENS) > 0x3fffffffLL)
        return fail(BN_ERR_UNSUPPORTED, "bn_attn_decode_paged: B * Hkv * max_seq_len is too large for one launch");
    if (pool_pages * Hkv * DEC_BOX_ROWS > 0x7fffffffLL)
        return fail(BN_ERR_UNSUPPORTED, "bn_attn_decode_paged: pool of %lld pages is too large", (long long)pool_pages);
    if ((reinterpret_cast<uintptr_t>(q) & 7) || (out && (reinterpret_cast<uintptr_t>(out) & 7)) ||
        (out_f32 && (reinterpret_cast<uintptr_t>(out_f32) & 15)))
        return fail(BN_ERR_INVALID_ARG, "bn_attn_decode_paged: q/out buffers must be 8/8/16-byte aligned");
    if (int rc = require_sm100()) return rc;
    if (B == 0) return BN_OK;
    const int min_tokens = pick_min_tokens(chunk_tokens);
    const DecodeLayout L = decode_layout(B, Hkv, max_seq_len, min_tokens, ticket_slots ? ticket_slots : regular_ticket_slots(Hkv));
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
    p.min_stages = min_tokens / DEC_STAGE_TOKENS;
    p.max_parts = L.max_parts;
    p.rope_q = rope_q;
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
    // no more CTAs than ranges of the minimum length can exist
    const long long max_ranges = (long long)B * Hkv * ((max_seq_len + min_tokens - 1) / min_tokens + 1);
    const int grid = (int)(max_ranges < sms ? (max_ranges > 0 ? max_ranges : 1) : sms);
    // Programmatic dependent launch: the kernel's set-up (barriers, tensor-map fetch) may overlap the tail of the
    // previous kernel of the stream; the kernel itself waits for that kernel's completion before it reads or
    // writes global memory.  If the attribute is refused, fall back to an ordinary launch.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(DEC_THREADS);
    cfg.dynamicSmemBytes = DEC_SMEM_BYTES;
    cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, decode_paged_kernel, tmap, p) != cudaSuccess) {
        (void)cudaGetLastError();
        decode_paged_kernel<<<grid, DEC_THREADS, DEC_SMEM_BYTES, as_stream(stream)>>>(tmap, p);
    }
    return launch_status("bn_attn_decode_paged");
}

extern "C" int bn_attn_decode_paged(const void* q, const void* pool, int64_t pool_pages, const int32_t* page_table,
                                    int max_pages, const int32_t* seq_lens, const int32_t* q_positions, void* out,
                                    float* out_f32, float* lse, int B, int Hq, int Hkv, int D, float scale,
                                    float theta, int rope_q, int max_seq_len, int chunk_tokens, void* workspace,
                                    size_t workspace_bytes, bn_stream_t stream) {
    return decode_launch(q, pool, pool_pages, page_table, max_pages, seq_lens, q_positions, out, out_f32, lse, B, Hq,
                         Hkv, D, scale, theta, rope_q, max_seq_len, chunk_tokens, workspace, workspace_bytes, 0, stream);
}

// ---------------------------------------------------------------------------
// Decode without a caller-supplied scratch buffer
// ---------------------------------------------------------------------------
// Scratch of the split-KV combine for callers that cannot allocate device memory.  The array lives in the
// library's device image: every GPU that loads the library holds these bytes until the process exits.
constexpr int DEC_STATIC_MAX_BG = 256;        // sequences x KV heads
constexpr int DEC_STATIC_MAX_SEQ_LEN = 4096;  // tokens per sequence
constexpr size_t DEC_STATIC_HEAD_BYTES = 256 + DEC_STATIC_MAX_BG * sizeof(int);   // header + tickets: the part that must start at zero
constexpr size_t DEC_STATIC_BYTES =
    DEC_STATIC_HEAD_BYTES +
    2 * (size_t)DEC_STATIC_MAX_BG * (DEC_STATIC_MAX_SEQ_LEN / DEC_DEFAULT_MIN_TOKENS + 2) * DEC_G * sizeof(float) +
    (size_t)DEC_STATIC_MAX_BG * (DEC_STATIC_MAX_SEQ_LEN / DEC_DEFAULT_MIN_TOKENS + 2) * DEC_G * DEC_D * sizeof(float);
static __device__ __align__(256) unsigned char g_decode_static_scratch[DEC_STATIC_BYTES];

// Device address of the built-in scratch on the current device.  The array's name is only a host-side handle, so
// the runtime is asked for the address, once per device and with that device current; that first time the header
// and the tickets are cleared on `stream`.
static int static_scratch(const char* who, bn_stream_t stream, void** out) {
    constexpr int kMaxDevices = 64;
    static void* s_scratch[kMaxDevices] = {};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return fail(BN_ERR_CUDA, "%s: cudaGetDevice: %s", who, cudaGetErrorString(e));
    void* scratch = s_scratch[dev];
    if (!scratch) {
        e = cudaGetSymbolAddress(&scratch, g_decode_static_scratch);
        if (e != cudaSuccess || !scratch)
            return fail(BN_ERR_CUDA, "%s: cudaGetSymbolAddress: %s", who, cudaGetErrorString(e));
        e = cudaMemsetAsync(scratch, 0, DEC_STATIC_HEAD_BYTES, as_stream(stream));
        if (e != cudaSuccess) return fail(BN_ERR_CUDA, "%s: cudaMemsetAsync: %s", who, cudaGetErrorString(e));
        s_scratch[dev] = scratch;
    }
    *out = scratch;
    return BN_OK;
}

extern "C" int bn_attn_decode_paged_static(const void* q, const void* pool, int64_t pool_pages,
                                           const int32_t* page_table, int max_pages, const int32_t* seq_lens,
                                           const int32_t* q_positions, void* out, float* out_f32, float* lse, int B,
                                           int Hq, int Hkv, int D, float scale, float theta, int rope_q,
                                           int max_seq_len, bn_stream_t stream) {
    if (B < 0 || Hkv <= 0 || max_seq_len < 0)
        return fail(BN_ERR_INVALID_ARG, "bn_attn_decode_paged_static: bad sizes B=%d Hkv=%d max_seq_len=%d", B, Hkv,
                    max_seq_len);
    if ((long long)B * Hkv > DEC_STATIC_MAX_BG || max_seq_len > DEC_STATIC_MAX_SEQ_LEN)
        return fail(BN_ERR_UNSUPPORTED,
                    "bn_attn_decode_paged_static: B*Hkv=%lld, max_seq_len=%d exceed the built-in scratch (B*Hkv <= %d, "
                    "max_seq_len <= %d); use bn_attn_decode_paged with a caller-owned buffer",
                    (long long)B * Hkv, max_seq_len, DEC_STATIC_MAX_BG, DEC_STATIC_MAX_SEQ_LEN);
    if (int rc = require_sm100()) return rc;
    void* scratch = nullptr;
    if (int rc = static_scratch("bn_attn_decode_paged_static", stream, &scratch)) return rc;
    // The ticket region always has DEC_STATIC_MAX_BG slots, so the partials start at the same byte for every
    // batch size and a call can never find an earlier call's partials where it expects zeroed tickets.
    return decode_launch(q, pool, pool_pages, page_table, max_pages, seq_lens, q_positions, out, out_f32, lse, B, Hq,
                         Hkv, D, scale, theta, rope_q, max_seq_len, 0, scratch, DEC_STATIC_BYTES, DEC_STATIC_MAX_BG,
                         stream);
}

extern "C" int bn_attn_decode_paged_static_status(bn_stream_t stream) {
    if (int rc = require_sm100()) return rc;
    void* scratch = nullptr;
    if (int rc = static_scratch("bn_attn_decode_paged_static_status", stream, &scratch)) return rc;
    int word = 0;
    cudaError_t e = cudaMemcpyAsync(&word, scratch, sizeof(word), cudaMemcpyDeviceToHost, as_stream(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(as_stream(stream));
    if (e != cudaSuccess) return fail(BN_ERR_CUDA, "bn_attn_decode_paged_static_status: %s", cudaGetErrorString(e));
    if (word != BN_ERR_TIMEOUT) return BN_OK;
    // a launch gave up half way: its tickets may be left non-zero, so header and tickets are cleared for the next call
    e = cudaMemsetAsync(scratch, 0, DEC_STATIC_HEAD_BYTES, as_stream(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(as_stream(stream));
    if (e != cudaSuccess) return fail(BN_ERR_CUDA, "bn_attn_decode_paged_static_status: %s", cudaGetErrorString(e));
    return fail(BN_ERR_TIMEOUT, "a bounded device-side wait ran out in a bn_attn_decode_paged_static call; its result "
                                "is invalid (the built-in scratch has been cleared for the next call)");
}

extern "C" int bn_attn_lse_combine_strided(const float* outs, int64_t outs_part_stride, const float* lses,
                                           int64_t lses_part_stride, int P, int64_t n, int D, float* out_f32,
                                           void* out_bf16, float* lse, bn_stream_t stream) {
    if (!outs || !lses || (!out_f32 && !out_bf16)) return fail(BN_ERR_INVALID_ARG, "bn_attn_lse_combine: null pointer");
    if (P <= 0 || n < 0 || D <= 0) return fail(BN_ERR_INVALID_ARG, "bn_attn_lse_combine: bad sizes P=%d D=%d", P, D);
    if (int rc = require_sm100()) return rc;
    if (n == 0) return BN_OK;
    lse_combine_kernel<<<(unsigned)n, 64, 0, as_stream(stream)>>>(outs, outs_part_stride, lses, lses_part_stride, P, n,
                                                                D, out_f32, static_cast<__nv_bfloat16*>(out_bf16), lse);
    return launch_status("bn_attn_lse_combine");
}

extern "C" int bn_attn_lse_combine(const float* outs, const float* lses, int P, int64_t n, int D, float* out_f32,
                                   void* out_bf16, float* lse, bn_stream_t stream) {
    return bn_attn_lse_combine_strided(outs, n * D, lses, n, P, n, D, out_f32, out_bf16, lse, stream);
}

// The one exchange step of the attention path: the log-sum-exp merge of the partial results of a sequence that is
// split across the GPUs of a node (long-context decode).  The reference is single-GPU (no NCCL, no peer access,
// no cudaSetDevice anywhere in its tree), so nothing here replaces reference code.
//
// Message: n rows of (D + 1) floats per rank (33.8 KB at batch 4 x 32 heads x (64 + 1)), i.e. latency-bound.  A
// collective library needs a launch for the all-gather and another for the merge; here ONE kernel per GPU does
// both over peer-mapped memory, and the data carries its own arrival flag:
//   phase 1  CTA t copies this rank's whole partial into the slot [parity][rank] of ONE rank's exchange buffer (the
//            t-th after its own, its own last) with plain 16-byte stores (NVLink peer stores; no multicast, no TMA),
//            each store = two floats and, beside each, the step number.  No fence and no counter: an 8-byte pair is
//            written as one piece, so a reader that sees the step number beside a value sees the value.
//   phase 2  every CTA merges the rows it owns in rank order (so every rank computes the same bits): it reads a row's
//            log-sum-exps and then its outputs from every rank's slot, again and again - with a time limit - until
//            the step number stands beside them.
// (The first two versions published with a system-scope fence and per-rank counters, every CTA storing a slice to
// every rank: 31 us at 8 GPUs; one CTA per target: 18 us; this form has no fence and no counter round trip at all.)
// Steps alternate between two slot sets: a rank can be at most one step ahead of another (it cannot finish step
// t + 1 before every rank has delivered step t + 1, which a rank does only after its own merge of step t), so the
// slots of step t are not overwritten before they have been read.  The step number only grows and a fresh buffer holds
// zeros, so a stale pair can never pass for the current step.
// A wait that runs out (a rank that never arrives) stores BN_ERR_TIMEOUT in the buffer's error word and the kernel
// returns; bn_exchange_status reports it.  After a timeout the exchange is out of step and must be destroyed.
#include "common.cuh"
#include "ptx.cuh"

namespace bn {

constexpr int EX_MAX_WORLD = 16;
constexpr int EX_CTAS = 8;         // fewest CTAs of a launch
constexpr int EX_THREADS = 256;
constexpr size_t EX_HEADER = 256;      // error word
constexpr size_t EX_FLAGS = 256;       // reserved

struct ExchangeParams {
    uint2* peer_slots[EX_MAX_WORLD];       // slot area of every rank's buffer (this rank's own: local pointer)
    int n_targets;                         // distinct buffers to deliver to (world, or 1 in single-process loop-back)
    const float* send;                     // this rank's partial: n * D outputs, then n log-sum-exps
    const uint2* slots;                    // own slot area: [2][world][n * (D + 1)] (value bits, step number)
    int* error_word;                       // header word 0; word 1 = steps completed, word 2 = CTAs done with this step
    float* out;
    float* lse;
    int world, rank, n, D;
    unsigned long long wait_ns;
};

__device__ __forceinline__ uint2 ld_pair(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// Values [idx] of every rank's slot, each read again until this step's number stands beside it (or the time limit runs
// out: false).  All first reads are issued before any is looked at.
template <int W>
__device__ __forceinline__ bool gather_pairs(const ExchangeParams& p, const uint2* base, size_t per_rank, size_t idx,
                                             unsigned active, uint32_t step, float (&val)[W], uint64_t t0, int* s_abort) {
    uint2 v[W];
#pragma unroll
    for (int r = 0; r < W; ++r)
        if ((active >> r) & 1u) v[r] = ld_pair(base + (size_t)r * per_rank + idx);
    for (uint32_t it = 0;; ++it) {
        bool all = true;
#pragma unroll
        for (int r = 0; r < W; ++r)
            if (((active >> r) & 1u) && v[r].y != step) {
                v[r] = ld_pair(base + (size_t)r * per_rank + idx);
                all = false;
            }
        if (all) break;
        if ((it & 63) == 63 && (*reinterpret_cast<volatile int*>(s_abort) || ptx::globaltimer_ns() - t0 > p.wait_ns)) {
            *reinterpret_cast<volatile int*>(s_abort) = 1;
            return false;
        }
    }
#pragma unroll
    for (int r = 0; r < W; ++r) val[r] = ((active >> r) & 1u) ? __uint_as_float(v[r].x) : 0.f;
    return true;
}

// 96 registers: a CTA of this kernel then fits beside a CTA of the decode kernel (124 registers x 320 threads), so
// as a programmatic dependent of it the kernel is resident, and waiting, when the decode kernel ends.
// W = the most ranks the instance handles (its per-rank values live in registers): 8 or EX_MAX_WORLD.
template <int W>
__global__ void __maxnreg__(96) exchange_merge_kernel(const ExchangeParams p) {
    __shared__ int s_abort;
    // nothing is read before the kernel that produced `send` has completed; the next kernel of the stream (the next
    // step's decode kernel) may begin its set-up while this one waits for the other ranks
    ptx::grid_dependency_wait();
    ptx::grid_launch_dependents();
    const size_t per_rank = (size_t)p.n * (p.D + 1);       // floats; a multiple of 4 (checked on the host)
    // The step number lives in the buffer, not in the launch: every CTA reads "steps completed" (the last CTA of the
    // previous launch wrote it; the wait above, or stream order, puts that before this read) - so the same launch can
    // be replayed from a CUDA graph.  It is advanced below by the last CTA to finish, when every CTA has read it.
    const uint32_t step = *reinterpret_cast<volatile uint32_t*>(p.error_word + 1) + 1u;     // 1, 2, ...
    const int parity = (int)(step & 1u);
    if (threadIdx.x == 0) s_abort = 0;
    __syncthreads();
    // ---- phase 1: CTA t delivers this rank's whole partial to ONE rank
    if ((int)blockIdx.x < p.n_targets) {
        const int r = (p.rank + 1 + (int)blockIdx.x) % p.n_targets;
        const float2* src = reinterpret_cast<const float2*>(p.send);
        uint4* dst = reinterpret_cast<uint4*>(p.peer_slots[r] + ((size_t)parity * p.world + p.rank) * per_rank);
        for (int v = threadIdx.x; v < (int)(per_rank / 2); v += EX_THREADS) {
            const float2 x = src[v];
            asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst + v), "r"(__float_as_uint(x.x)),
                         "r"(step), "r"(__float_as_uint(x.y)), "r"(step)
                         : "memory");
        }
    }
    // ---- phase 2: merge the rows this CTA owns, parts in rank order
    const uint64_t t0 = ptx::globaltimer_ns();
    const uint2* base = p.slots + (size_t)parity * p.world * per_rank;
    const unsigned all_ranks = p.world >= 32 ? 0xffffffffu : ((1u << p.world) - 1u);
    const int sub = threadIdx.x / 64, lane = threadIdx.x % 64;      // four rows at a time, 64 threads each
    bool ok = true;
    for (int row = blockIdx.x * 4 + sub; ok && row < p.n; row += gridDim.x * 4) {
        float l[W], wgt[W];
        ok = gather_pairs<W>(p, base, per_rank, (size_t)p.n * p.D + row, all_ranks, step, l, t0, &s_abort);
        if (!ok) break;
        float mstar = -INFINITY;
        unsigned holds = 0;                         // ranks that hold a token of the row
#pragma unroll
        for (int r = 0; r < W; ++r)
            if (r < p.world) {
                mstar = fmaxf(mstar, l[r]);
                if (l[r] > -INFINITY) holds |= 1u << r;
            }
        const float ms = mstar == -INFINITY ? 0.f : mstar;
        float tot = 0.f;
#pragma unroll
        for (int r = 0; r < W; ++r) {
            wgt[r] = r < p.world ? expf(l[r] - ms) : 0.f;       // 0 for a rank that holds no token of the row
            if (r < p.world) tot += wgt[r];                     // in rank order: every rank computes the same bits
        }
        const float inv = tot > 0.f ? 1.f / tot : 0.f;
        for (int d = lane; d < p.D; d += 64) {
            float o[W];
            // every rank's value is waited for, also where its weight is 0: the slot must be complete before the step ends
            ok = gather_pairs<W>(p, base, per_rank, (size_t)row * p.D + d, all_ranks, step, o, t0, &s_abort);
            if (!ok) break;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < W; ++r)
                if ((holds >> r) & 1u) acc += o[r] * wgt[r];
            p.out[(size_t)row * p.D + d] = acc * inv;
        }
        if (ok && p.lse && lane == 0) p.lse[row] = tot > 0.f ? ms + logf(tot) : -INFINITY;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (s_abort) atomicExch(p.error_word, BN_ERR_TIMEOUT);
        __threadfence();
        if (atomicAdd(p.error_word + 2, 1) == (int)gridDim.x - 1) {      // the last CTA of the launch
            p.error_word[2] = 0;
            *reinterpret_cast<volatile uint32_t*>(p.error_word + 1) = step;
        }
    }
}

}  // namespace bn

using namespace bn;

struct bn_exchange {
    int n, D, world, rank;
    int step;
    int n_targets;
    void* buffer;                      // header | counters | slots
    size_t bytes;
    void* peer_base[EX_MAX_WORLD];     // mapped peer buffers (NULL for ourselves / not opened)
    bool opened;
};

static size_t exchange_bytes(int n, int D, int world) {
    return EX_HEADER + EX_FLAGS + (size_t)2 * world * n * (D + 1) * sizeof(uint2);
}

extern "C" int bn_exchange_create(int n, int D, int world, int rank, bn_exchange_t** out) {
    if (!out) return fail(BN_ERR_INVALID_ARG, "bn_exchange_create: null pointer");
    if (n <= 0 || D <= 0 || world <= 0 || world > EX_MAX_WORLD || rank < 0 || rank >= world)
        return fail(BN_ERR_INVALID_ARG, "bn_exchange_create: bad sizes n=%d D=%d world=%d rank=%d (world <= %d)", n, D, world,
                    rank, EX_MAX_WORLD);
    if ((n * (D + 1)) % 4)
        return fail(BN_ERR_UNSUPPORTED, "bn_exchange_create: n * (D + 1) = %d must be a multiple of 4", n * (D + 1));
    if (int rc = require_sm100()) return rc;
    bn_exchange* x = new bn_exchange();
    x->n = n; x->D = D; x->world = world; x->rank = rank; x->step = 0; x->n_targets = 0; x->opened = false;
    for (int i = 0; i < EX_MAX_WORLD; ++i) x->peer_base[i] = nullptr;
    x->bytes = exchange_bytes(n, D, world);
    cudaError_t e = cudaMalloc(&x->buffer, x->bytes);
    if (e == cudaSuccess) e = cudaMemset(x->buffer, 0, x->bytes);
    if (e != cudaSuccess) {
        delete x;
        return fail(BN_ERR_CUDA, "bn_exchange_create: %s", cudaGetErrorString(e));
    }
    *out = x;
    return BN_OK;
}

extern "C" int bn_exchange_ipc_handle(bn_exchange_t* x, void* handle64) {
    if (!x || !handle64) return fail(BN_ERR_INVALID_ARG, "bn_exchange_ipc_handle: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, x->buffer);
    if (e != cudaSuccess) return fail(BN_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    memcpy(handle64, &h, 64);
    return BN_OK;
}

extern "C" int bn_exchange_open_peers(bn_exchange_t* x, const void* handles, int loopback) {
    if (!x) return fail(BN_ERR_INVALID_ARG, "bn_exchange_open_peers: null pointer");
    if (x->opened) return fail(BN_ERR_INVALID_ARG, "bn_exchange_open_peers: already opened");
    if (loopback) {             // single process: every "peer" is this buffer, which then receives our step only
        x->n_targets = 1;
        x->opened = true;
        return BN_OK;
    }
    if (!handles) return fail(BN_ERR_INVALID_ARG, "bn_exchange_open_peers: null handles");
    for (int r = 0; r < x->world; ++r) {
        if (r == x->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const char*>(handles) + (size_t)r * 64, 64);
        cudaError_t e = cudaIpcOpenMemHandle(&x->peer_base[r], h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int q = 0; q < r; ++q)
                if (x->peer_base[q]) { cudaIpcCloseMemHandle(x->peer_base[q]); x->peer_base[q] = nullptr; }
            return fail(BN_ERR_CUDA, "cudaIpcOpenMemHandle(rank %d): %s", r, cudaGetErrorString(e));
        }
    }
    x->n_targets = x->world;
    x->opened = true;
    return BN_OK;
}

extern "C" int bn_exchange_combine(bn_exchange_t* x, const float* partial, float* out, float* lse, unsigned wait_us,
                                   bn_stream_t stream) {
    if (!x || !partial || !out) return fail(BN_ERR_INVALID_ARG, "bn_exchange_combine: null pointer");
    if (!x->opened) return fail(BN_ERR_INVALID_ARG, "bn_exchange_combine: peers not opened");
    if (reinterpret_cast<uintptr_t>(partial) & 15) return fail(BN_ERR_INVALID_ARG, "bn_exchange_combine: partial must be 16-byte aligned");
    ExchangeParams p;
    char* own = static_cast<char*>(x->buffer);
    for (int r = 0; r < EX_MAX_WORLD; ++r) p.peer_slots[r] = nullptr;
    for (int r = 0; r < x->n_targets; ++r) {
        char* base = (r == x->rank || x->n_targets == 1) ? own : static_cast<char*>(x->peer_base[r]);
        p.peer_slots[r] = reinterpret_cast<uint2*>(base + EX_HEADER + EX_FLAGS);
    }
    p.n_targets = x->n_targets;
    p.send = partial;
    p.slots = reinterpret_cast<const uint2*>(own + EX_HEADER + EX_FLAGS);
    p.error_word = reinterpret_cast<int*>(own);
    p.out = out;
    p.lse = lse;
    p.world = x->world; p.rank = x->rank; p.n = x->n; p.D = x->D;
    p.wait_ns = (unsigned long long)(wait_us ? wait_us : 1000000u) * 1000ull;
    // one CTA merges four rows at a time; enough CTAs that every row group is merged in the first pass (a pass is two
    // round trips to L2), and at least one CTA per target rank for the delivery
    int want = (x->n + 3) / 4;
    if (want > 128) want = 128;
    if (want < EX_CTAS) want = EX_CTAS;
    const unsigned grid = (unsigned)(x->n_targets > want ? x->n_targets : want);
    if (x->world <= 8) launch_dependent(exchange_merge_kernel<8>, grid, EX_THREADS, 0, as_stream(stream), p);
    else launch_dependent(exchange_merge_kernel<EX_MAX_WORLD>, grid, EX_THREADS, 0, as_stream(stream), p);
    return launch_status("bn_exchange_combine");
}

extern "C" int bn_exchange_status(bn_exchange_t* x, bn_stream_t stream) {
    if (!x) return fail(BN_ERR_INVALID_ARG, "bn_exchange_status: null pointer");
    int word = 0;
    cudaError_t e = cudaMemcpyAsync(&word, x->buffer, sizeof(word), cudaMemcpyDeviceToHost, as_stream(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(as_stream(stream));
    if (e != cudaSuccess) return fail(BN_ERR_CUDA, "bn_exchange_status: %s", cudaGetErrorString(e));
    if (word == BN_ERR_TIMEOUT)
        return fail(BN_ERR_TIMEOUT, "a rank did not deliver its partial results in time; the exchange is out of step and "
                                    "must be destroyed");
    return BN_OK;
}

extern "C" void bn_exchange_destroy(bn_exchange_t* x) {
    if (!x) return;
    for (int r = 0; r < EX_MAX_WORLD; ++r)
        if (x->peer_base[r]) cudaIpcCloseMemHandle(x->peer_base[r]);
    cudaFree(x->buffer);
    delete x;
}

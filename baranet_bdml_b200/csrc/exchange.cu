// The one exchange step of the attention path: the log-sum-exp merge of the partial results of a sequence that is
// split across the GPUs of a node (long-context decode).  The reference is single-GPU (no NCCL, no peer access,
// no cudaSetDevice anywhere in its tree), so nothing here replaces reference code.
//
// Message: n rows of (D + 1) floats per rank (33.8 KB at batch 4 x 32 heads x (64 + 1)), i.e. latency-bound.  A
// collective library needs a launch for the all-gather and another for the merge; here ONE kernel per GPU does
// both over peer-mapped memory:
//   phase 1  every CTA copies its slice of this rank's partial into the slot [parity][rank] of EVERY rank's
//            exchange buffer with plain 16-byte stores (NVLink peer stores; no multicast, no TMA), fences at system
//            scope and adds 1 to the counter [rank] in each of those buffers;
//   phase 2  it waits, with a time limit, until the counters of its own buffer show that every CTA of every rank
//            has delivered this step, then merges the rows it owns in rank order (so every rank computes the same
//            bits) and writes them out.
// Steps alternate between two slot sets: a rank can be at most one step ahead of another (it cannot finish step
// t + 1 before every rank has delivered step t + 1, which a rank does only after its own merge of step t), so the
// slots of step t are not overwritten before they have been read.  The counters only grow (step e expects
// e * CTAs per rank), so nothing is ever reset between steps.
// A wait that runs out (a rank that never arrives) stores BN_ERR_TIMEOUT in the buffer's error word and the kernel
// returns; bn_exchange_status reports it.  After a timeout the exchange is out of step and must be destroyed.
#include "common.cuh"
#include "ptx.cuh"

namespace bn {

constexpr int EX_MAX_WORLD = 16;
constexpr int EX_CTAS = 8;
constexpr int EX_THREADS = 256;
constexpr size_t EX_HEADER = 256;      // error word
constexpr size_t EX_FLAGS = 256;       // EX_MAX_WORLD counters

struct ExchangeParams {
    float* peer_slots[EX_MAX_WORLD];       // slot area of every rank's buffer (this rank's own: local pointer)
    int* peer_flags[EX_MAX_WORLD];
    int n_targets;                         // distinct buffers to deliver to (world, or 1 in single-process loop-back)
    const float* send;                     // this rank's partial: n * D outputs, then n log-sum-exps
    float* slots;                          // own slot area: [2][world][n * (D + 1)]
    volatile int* flags;                   // own counters
    int* error_word;
    float* out;
    float* lse;
    int world, rank, n, D;
    int expect;                            // counter value that means "delivered": the step number
    int parity;
    unsigned long long wait_ns;
};

// 96 registers: a CTA of this kernel then fits beside a CTA of the decode kernel (124 registers x 320 threads), so
// as a programmatic dependent of it the kernel is resident, and waiting, when the decode kernel ends.
__global__ void __maxnreg__(96) exchange_merge_kernel(const ExchangeParams p) {
    __shared__ int s_abort;
    // nothing is read before the kernel that produced `send` has completed; the next kernel of the stream (the next
    // step's decode kernel) may begin its set-up while this one waits for the other ranks
    ptx::grid_dependency_wait();
    ptx::grid_launch_dependents();
    const int per_rank = p.n * (p.D + 1);                  // floats; a multiple of 4 (checked on the host)
    const int n_vec = per_rank / 4;
    if (threadIdx.x == 0) s_abort = 0;
    // ---- phase 1: CTA t delivers this rank's whole partial to ONE rank (the t-th after ourselves, ourselves last), so
    // a step costs every rank one system-scope fence and one counter update per target, whatever the number of CTAs
    if ((int)blockIdx.x < p.n_targets) {
        const int r = (p.rank + 1 + (int)blockIdx.x) % p.n_targets;
        const float4* src = reinterpret_cast<const float4*>(p.send);
        float4* dst = reinterpret_cast<float4*>(p.peer_slots[r] + ((size_t)p.parity * p.world + p.rank) * per_rank);
        for (int v = threadIdx.x; v < n_vec; v += EX_THREADS) dst[v] = src[v];
        // the CTA barrier orders every thread's stores before the one thread that publishes them: only it executes the
        // system-scope fence (cumulative over what the barrier made visible to it)
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence_system();
            atomicAdd_system(p.peer_flags[r] + p.rank, 1);
        }
    }
    // ---- phase 2: everybody's step has arrived in OUR buffer?
    if ((int)threadIdx.x < p.world) {
        const uint64_t t0 = ptx::globaltimer_ns();
        for (uint32_t it = 0;; ++it) {
            if (p.flags[threadIdx.x] - p.expect >= 0) break;       // counters only grow
            if ((it & 63) == 63) {
                if (s_abort || ptx::globaltimer_ns() - t0 > p.wait_ns) { s_abort = 1; break; }
            }
        }
        __threadfence_system();      // acquire side, by the threads that saw the counters; the barrier hands it on
    }
    __syncthreads();
    if (s_abort) {
        if (threadIdx.x == 0) atomicExch(p.error_word, BN_ERR_TIMEOUT);
        return;
    }
    // ---- merge the rows this CTA owns, parts in rank order
    const float* base = p.slots + (size_t)p.parity * p.world * per_rank;
    const int sub = threadIdx.x / 64, lane = threadIdx.x % 64;      // four rows at a time, 64 threads each
    for (int row = blockIdx.x * 4 + sub; row < p.n; row += gridDim.x * 4) {
        // every rank's log-sum-exp of the row first (independent loads: one round trip to L2, not one per rank), then
        // the weights e^(l_r - m*) once, then the rank's O values, again all requested before the first use
        float l[EX_MAX_WORLD], wgt[EX_MAX_WORLD];
#pragma unroll
        for (int r = 0; r < EX_MAX_WORLD; ++r)
            l[r] = r < p.world ? __ldcg(base + (size_t)r * per_rank + (size_t)p.n * p.D + row) : -INFINITY;
        float mstar = -INFINITY;
#pragma unroll
        for (int r = 0; r < EX_MAX_WORLD; ++r) mstar = fmaxf(mstar, l[r]);
        const float ms = mstar == -INFINITY ? 0.f : mstar;
        float tot = 0.f;
#pragma unroll
        for (int r = 0; r < EX_MAX_WORLD; ++r) {
            wgt[r] = expf(l[r] - ms);               // 0 for a rank that holds no token of the row
            if (r < p.world) tot += wgt[r];         // in rank order: every rank computes the same bits
        }
        const float inv = tot > 0.f ? 1.f / tot : 0.f;
        for (int d = lane; d < p.D; d += 64) {
            float o[EX_MAX_WORLD];
#pragma unroll
            for (int r = 0; r < EX_MAX_WORLD; ++r)
                o[r] = (r < p.world && l[r] > -INFINITY) ? __ldcg(base + (size_t)r * per_rank + (size_t)row * p.D + d) : 0.f;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < EX_MAX_WORLD; ++r)
                if (r < p.world && l[r] > -INFINITY) acc += o[r] * wgt[r];
            p.out[(size_t)row * p.D + d] = acc * inv;
        }
        if (p.lse && lane == 0) p.lse[row] = tot > 0.f ? ms + logf(tot) : -INFINITY;
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
    return EX_HEADER + EX_FLAGS + (size_t)2 * world * n * (D + 1) * sizeof(float);
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
    for (int r = 0; r < EX_MAX_WORLD; ++r) { p.peer_slots[r] = nullptr; p.peer_flags[r] = nullptr; }
    for (int r = 0; r < x->n_targets; ++r) {
        char* base = (r == x->rank || x->n_targets == 1) ? own : static_cast<char*>(x->peer_base[r]);
        p.peer_flags[r] = reinterpret_cast<int*>(base + EX_HEADER);
        p.peer_slots[r] = reinterpret_cast<float*>(base + EX_HEADER + EX_FLAGS);
    }
    p.n_targets = x->n_targets;
    p.send = partial;
    p.slots = reinterpret_cast<float*>(own + EX_HEADER + EX_FLAGS);
    p.flags = reinterpret_cast<volatile int*>(own + EX_HEADER);
    p.error_word = reinterpret_cast<int*>(own);
    p.out = out;
    p.lse = lse;
    p.world = x->world; p.rank = x->rank; p.n = x->n; p.D = x->D;
    x->step += 1;
    p.expect = x->step;                       // one delivery per source rank and step
    p.parity = x->step & 1;
    p.wait_ns = (unsigned long long)(wait_us ? wait_us : 1000000u) * 1000ull;
    launch_dependent(exchange_merge_kernel, (unsigned)(x->n_targets > EX_CTAS ? x->n_targets : EX_CTAS), EX_THREADS, 0,
                     as_stream(stream), p);
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

/*
 * bn_attn.h — C ABI of the B200 (sm_100a) fused grouped-query-attention module.
 *
 * Drop-in boundary for BareNet's attention hot path.  Every entry point takes
 * plain device pointers, element strides and sizes, launches on the given CUDA
 * stream (pass 0 for the legacy default stream that all of the reference's
 * operators use) and returns a status code; nothing here allocates device
 * memory, synchronises the device or owns a buffer.  There is no CPU fallback:
 * on a device that is not compute capability 10.x every call returns
 * BN_ERR_ARCH.
 *
 * Reference interfaces replaced (paths relative to the reference project):
 *   op_mm              src/ops/op_mm.cuh:39-57, op_mm_optimized.cuh:73-87
 *   op_rope            src/ops/op_rope.cuh:101-126
 *   op_multiply(t, c)  src/ops/op_elemwise.cuh:436-451
 *   op_softmax         src/ops/op_softmax.cuh:153-180
 *   op_attention_fused src/ops/op_attention_fused.cuh:109-138  (the operator
 *                      slot: same argument meaning, never bound upstream)
 *   the op sequence of GroupedQueryAttention.__call__
 *                      mygrad/llama/llama_layers.py:161-183
 *   decode semantics   mygrad/llama/llama_model.py:136-144
 *
 * Conventions: bf16 buffers are passed as `const void*` / `void*` holding
 * IEEE bfloat16 bit patterns; "elements" in a stride means elements of the
 * buffer's own type.
 */
#ifndef BN_ATTN_H_
#define BN_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes (0 = success).  A binding converts non-zero into the
 * reference's error convention, std::runtime_error(bn_last_error())
 * (src/utils/check_error.cuh:8-14). */
#define BN_OK 0
#define BN_ERR_INVALID_ARG 1   /* null pointer, negative size, misaligned buffer */
#define BN_ERR_UNSUPPORTED 2   /* shape outside what the kernels are built for */
#define BN_ERR_CUDA 3          /* a CUDA runtime/driver call failed */
#define BN_ERR_ARCH 4          /* current device is not sm_100 */
#define BN_ERR_TIMEOUT 5       /* a bounded device-side wait ran out */
#define BN_ERR_WORKSPACE 6     /* workspace missing or too small */

/* head modes of the fp32 prefill path */
#define BN_HEADS_COLLAPSED 0   /* the reference's semantics: ONE softmax over scores summed over all heads */
#define BN_HEADS_PER_HEAD 1    /* standard GQA: one softmax per query head, KV head = q_head / (Hq/Hkv) */

/* tokens per KV-cache page */
#define BN_PAGE_TOKENS 16

typedef void* bn_stream_t; /* a cudaStream_t */

/* exported symbol (the library is built with hidden default visibility) */
#if defined(__GNUC__)
#define BN_API __attribute__((visibility("default")))
#else
#define BN_API
#endif

/* Message of the last non-zero status returned on the calling thread. */
BN_API const char* bn_last_error(void);

/* Library version (major*100 + minor). */
BN_API int bn_version(void);

/* Every device-side wait in these kernels is bounded; a kernel that gave up
 * raises an error word at the head of the scratch buffer it was given.  This
 * call waits for `stream`, reads that word and returns BN_OK or
 * BN_ERR_TIMEOUT.  (It synchronises; use it in tests and after a suspected
 * hang, not on the hot path.)  After BN_ERR_TIMEOUT the scratch buffer must be
 * zero-filled again before reuse. */
BN_API int bn_workspace_status(const void* workspace, bn_stream_t stream);

/* Self-test of that mechanism (no counterpart in the reference): launches a small kernel whose only wait is for a
 * barrier that nothing arrives at, with a limit of limit_us microseconds (1..100000).  The wait gives up, the kernel
 * stores BN_ERR_TIMEOUT in the error word at the head of `workspace` (any scratch buffer of this library, or 4
 * zeroed bytes) and returns; bn_workspace_status then reports it.  The GPU is never hung or faulted by it. */
BN_API int bn_selftest_wait_timeout(void* workspace, unsigned limit_us, bn_stream_t stream);

/* ------------------------------------------------------------------------
 * fp32 path (bit-faithful to the reference's operator arithmetic)
 * ------------------------------------------------------------------------ */

/* C(M,N) = A(M,K) @ B(K,N), fp32, arbitrary element strides (so transposed and
 * sliced views work).  Each output is one fused-multiply-add chain with k
 * ascending, the order of the reference's kernels.
 * Replaces op_mm (src/ops/op_mm.cuh:39-57). */
BN_API int bn_mm_f32(const float* A, int64_t a_rs, int64_t a_cs, const float* B, int64_t b_rs, int64_t b_cs,
              float* C, int64_t c_rs, int64_t c_cs, int M, int K, int N, bn_stream_t stream);

/* y = RoPE(x): adjacent pairs (2i, 2i+1) inside every head_dim-wide column
 * block, row r at position r + position_offset, fp32 angles.
 * Replaces op_rope (src/ops/op_rope.cuh:101-126). */
BN_API int bn_rope_f32(const float* x, int64_t x_rs, int64_t x_cs, float* y, int64_t y_rs, int64_t y_cs, int rows,
                int cols, int head_dim, float theta, int position_offset, bn_stream_t stream);

/* out[i, :] = table[ids[i], :] on the device (fp32 rows, element row strides).  An id >= vocab yields a zero row
 * and BN_ERR_INVALID_ARG in *error_word (device int, may be NULL).
 * Replaces LLaMAModel.embed (mygrad/llama/llama_model.py:58-78), which copies the whole table to the host, gathers
 * there row by row and uploads the result. */
BN_API int bn_embedding_gather_f32(const float* table, int64_t table_rs, const uint32_t* ids, float* out,
                                   int64_t out_rs, int n_ids, int hidden, int vocab, int* error_word,
                                   bn_stream_t stream);

/* out[r] = index of the first maximum of row r of x (rows, cols) fp32 with element strides: element 0 stands unless
 * a later element is strictly greater, so ties keep the first index and a NaN wins only at index 0.
 * Replaces op_argmax (src/ops/op_reduction.cuh:196-210, MaxAccumFunc :5-19; TensorF.argmax,
 * src/py_tensor_shim.hh:220-224), for greedy decoding on the device instead of downloading the logits
 * (mygrad/llama/llama_model.py:136-160). */
BN_API int bn_argmax_rows_f32(const float* x, int64_t x_rs, int64_t x_cs, uint32_t* out, int rows, int cols,
                              bn_stream_t stream);

/* C (M,N) bf16 = A (M,K) bf16 @ Bt (N,K)^T bf16, fp32 accumulation (tcgen05 tensor cores, accumulators in tensor
 * memory).  Dense row-major operands; Bt is the weight stored transposed, (out_features, in_features), so both
 * operands are contiguous along K.  N and K multiples of 8, pointers 16-byte aligned; M, N, K otherwise free.
 * `error_word` (device int, may be NULL) receives BN_ERR_TIMEOUT if a bounded device-side wait runs out.
 * The projection GEMMs of the attention layer on bf16 operands: q/k/v/o_proj, `hidden_states @ W`
 * (mygrad/llama/llama_layers.py:157-159,186), reference operator op_mm (src/ops/op_mm.cuh:39-57), whose fp32
 * bit-compatible replacement is bn_mm_f32 above. */
BN_API int bn_gemm_bf16_nt(const void* a, const void* bt, void* c, int M, int N, int K, int* error_word,
                           bn_stream_t stream);

/* The same product for FEW rows (M <= 128 is where it pays: one token per sequence in a decode step), where the
 * weight matrix has to be streamed by all SMs: 64-wide N tiles and the K range cut into up to 8 parts, fp32 partial
 * sums in `workspace`, added in a fixed order by a second small kernel (results do not depend on timing).
 * workspace: bn_gemm_bf16_nt_small_m_workspace_bytes(M, N, K) bytes, 16-byte aligned; contents need not be kept. */
BN_API size_t bn_gemm_bf16_nt_small_m_workspace_bytes(int M, int N, int K);
BN_API int bn_gemm_bf16_nt_small_m(const void* a, const void* bt, void* c, int M, int N, int K, void* workspace,
                                   size_t workspace_bytes, int* error_word, bn_stream_t stream);

/* The same product for M <= 16 rows (a decode step with up to 16 sequences on the GPU): the weight matrix streamed
 * through all SMs with warp-level MMAs (mma.sync m16n8k16, whose M is the whole batch) - no scratch, one launch.
 * The N columns may go to up to three outputs: columns [0, n0) to out0 (M, n0), [n0, n0 + n1) to out1 (M, n1), the
 * rest to out2 - the q, k and v projections of the layer as one launch over the concatenated weight.  For a plain
 * product pass n0 = N, n1 = 0, out1 = out2 = NULL.  K a multiple of 256 (<= 8192), N, n0, n1 multiples of 8.
 * bn_gemm_swiglu_bf16_nt_skinny: h (M, inter) = silu(x @ gate) * (x @ up) with the two weights given separately,
 * (inter, K) each (not the packed form of bn_gemm_swiglu_bf16_nt). */
BN_API int bn_gemm_bf16_nt_skinny(const void* a, const void* bt, int M, int N, int K, void* out0, int n0, void* out1,
                                  int n1, void* out2, bn_stream_t stream);
BN_API int bn_gemm_swiglu_bf16_nt_skinny(const void* x, const void* gate_t, const void* up_t, void* h, int M, int inter,
                                         int K, bn_stream_t stream);

/* The q, k and v projections of a decode step (one new token per row, M <= 16) with the cache append in the same launch:
 * x (M, hidden) @ wqkv_t ((Hq + 2 Hkv) D, hidden)^T; the q columns go to q_out (M, Hq D), the k columns are rotated at
 * positions[row] and written with the v columns into the page of (seq_ids[row], positions[row]) - the bits that
 * bn_gemm_bf16_nt_skinny followed by bn_kv_append (bf16 rows) leave in the cache, in one launch instead of two
 * (mygrad/llama/llama_layers.py:157-171 for the new token only).  Cache arguments as bn_kv_append; rows whose position
 * or page is out of range are skipped as there.  hidden a multiple of 256 (<= 8192), D a multiple of 8. */
BN_API int bn_gemm_qkv_append_bf16_skinny(const void* x, const void* wqkv_t, int M, int hidden, int Hq, int Hkv, int D,
                                          void* q_out, void* pool, int64_t pool_pages, const int32_t* page_table,
                                          int max_pages, const int32_t* seq_ids, const int32_t* positions, float theta,
                                          bn_stream_t stream);

/* h (M, inter) bf16 = silu(x @ Wgate) * (x @ Wup): both GEMMs of the SwiGLU MLP, the activation and the product in
 * one launch of the tensor-core GEMM.  x (M,K) bf16; gate_up_t is the PACKED weight, ceil(inter/128)*256 rows of K
 * bf16: for every block of 128 intermediate indices, the 128 rows of Wgate^T followed by the 128 rows of Wup^T for
 * the same indices (rows beyond `inter` zero).  inter and K multiples of 8.
 * Replaces `gate = x @ gate_proj; gate = gate.silu(); up = x @ up_proj; inter = gate * up` of MLP.__call__
 * (mygrad/llama/llama_layers.py:217-228; op_mm, op_silu src/ops/op_silu.cuh:7-15, op_multiply); the down projection
 * that follows is bn_gemm_bf16_nt. */
BN_API int bn_gemm_swiglu_bf16_nt(const void* x, const void* gate_up_t, void* h, int M, int inter, int K,
                                  int* error_word, bn_stream_t stream);

/* y = x / sqrt(mean(x^2) + eps) * w, row by row; x, y (rows, hidden), w (hidden) with element strides.
 * Same arithmetic order as the reference kernel (256 partial fused-multiply-add chains, its reduction tree, IEEE
 * division and square root), so the result is the reference's bit for bit.
 * Replaces op_rmsnorm (src/ops/op_rmsnorm.cuh:8-53, launcher :134-157; bound as TensorF.rmsnorm,
 * src/py_tensor_shim.hh:256-260). */
BN_API int bn_rmsnorm_f32(const float* x, int64_t x_rs, int64_t x_cs, const float* w, int64_t w_cs, float* y,
                          int64_t y_rs, int64_t y_cs, int rows, int hidden, float eps, bn_stream_t stream);

/* sum = a + b (fp32), y = rmsnorm(sum) in one pass; `sum` may be NULL when the caller does not need it.
 * Replaces the pair op_add + op_rmsnorm that LLaMADecoderLayer runs around attention and the MLP
 * (`hidden = residual + hidden; hidden = norm(hidden)`, mygrad/llama/llama_layers.py:279-283), which writes the
 * sum and reads it back; bit-identical to that pair.  (The reference's own fused kernel, op_rmsnorm_residual,
 * src/ops/op_mm_optimized.cuh:93-162, computes norm(x)*w + residual instead and is never called.) */
BN_API int bn_add_rmsnorm_f32(const float* a, int64_t a_rs, int64_t a_cs, const float* b, int64_t b_rs, int64_t b_cs,
                              const float* w, int64_t w_cs, float* sum, int64_t s_rs, int64_t s_cs, float* y,
                              int64_t y_rs, int64_t y_cs, int rows, int hidden, float eps, bn_stream_t stream);

/* The same pair on a bf16 residual stream (rows, hidden) bf16, dense: sum = a + b rounded to bf16 (b may be NULL:
 * sum = a), y = sum / sqrt(mean(sum^2) + eps) * w computed in fp32 and rounded once.  `sum` may be NULL.  hidden a
 * multiple of 8, pointers 16-byte aligned.  Used by the bf16 decoder layer (RMSNorm and the residual adds of
 * LLaMADecoderLayer, mygrad/llama/llama_layers.py:262-287, on bf16 activations). */
BN_API int bn_add_rmsnorm_bf16(const void* a, const void* b, const void* w, void* sum, void* y, int rows, int hidden,
                               float eps, bn_stream_t stream);

/* Fused attention core, fp32:
 *   out = softmax_causal((rope(q) @ repeat(rope(k))^T) * scale) @ repeat(v)
 * q, out: (S, Hq*D); k, v: (S, Hkv*D); all with element strides.
 * heads_mode BN_HEADS_COLLAPSED reproduces the reference layer exactly (one
 * (S,S) score matrix over the full Hq*D width, one softmax); BN_HEADS_PER_HEAD
 * applies the same operators per D-wide head.  causal: key j valid iff
 * j <= row + position_offset (src/ops/op_softmax.cuh:88-101).  apply_rope = 0
 * skips the rotation (inputs already rotated).  No workspace is needed.
 * Takes the slot of op_attention_fused (src/ops/op_attention_fused.cuh:109-118)
 * and replaces llama_layers.py:161-183. */
BN_API int bn_attn_prefill_f32(const float* q, int64_t q_rs, int64_t q_cs, const float* k, int64_t k_rs, int64_t k_cs,
                        const float* v, int64_t v_rs, int64_t v_cs, float* out, int64_t o_rs, int64_t o_cs,
                        int S, int Hq, int Hkv, int D, float scale, float theta, int position_offset, int causal,
                        int heads_mode, int apply_rope, bn_stream_t stream);

/* ------------------------------------------------------------------------
 * bf16 path (fp32 accumulation), per-head GQA
 * ------------------------------------------------------------------------ */

/* Bytes of scratch bn_attn_prefill_bf16 needs for this shape. */
BN_API size_t bn_attn_prefill_bf16_workspace_bytes(int B, int S, int Hq, int Hkv, int D);

/* Causal (or full) prefill attention with RoPE fused.
 *   q   (B, S, Hq,  D) bf16, pre-RoPE       out (B, S, Hq, D) bf16
 *   k,v (B, S, Hkv, D) bf16, k pre-RoPE     lse (B, Hq, S) fp32 natural log, may be NULL
 * Row s sits at position s + position_offset; key j is valid iff
 * j <= s + position_offset when causal.  D must be 64.  The same math as
 * bn_attn_prefill_f32 in BN_HEADS_PER_HEAD mode on bf16 operands.
 * Two launches: K is rotated once into the scratch buffer (it is read by every
 * query head of its group and every query tile), then the attention kernel
 * (tcgen05 tensor cores, TMEM accumulators, TMA-staged K/V) runs.
 * flags: 0, or BN_PREFILL_REUSE_ROTATED_K when the scratch buffer still holds
 * the rotated K of an earlier call on the same k / position_offset, or the one
 * written by bn_gemm_qkv_rope_bf16 (skips the first launch; k may then be NULL).
 * BN_PREFILL_SINGLE_TILE_KERNEL selects the simpler kernel variant (one query
 * tile per CTA, two CTAs per SM) kept for comparison. */
#define BN_PREFILL_REUSE_ROTATED_K 0x100
#define BN_PREFILL_SINGLE_TILE_KERNEL 0x200
BN_API int bn_attn_prefill_bf16(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int Hq,
                         int Hkv, int D, float scale, float theta, int position_offset, int causal, int flags,
                                void* workspace, size_t workspace_bytes, bn_stream_t stream);

/* The q, k and v projections of the layer as ONE tensor-core GEMM with RoPE(K), the cache append and the K operand
 * of the attention kernel produced in its epilogue (mygrad/llama/llama_layers.py:157-163: three op_mm launches and
 * the K rotation; plus what bn_kv_append does):
 *   x (B*S, hidden) bf16; wqkv_t ((Hq + 2*Hkv) * D, hidden) bf16 = the rows of Wq^T, Wk^T, Wv^T one after the other;
 *   q_out (B, S, Hq, D) bf16 as projected (bn_attn_prefill_bf16 rotates Q itself); v_out (B, S, Hkv, D) bf16;
 *   rotated K (from the fp32 accumulators: one rounding) and the per-tile key norms go into `prefill_workspace`,
 *   the scratch buffer of bn_attn_prefill_bf16 for the same B, S, Hkv, whose cos/sin table must have been written
 *   by bn_attn_prefill_bf16_table (or by an earlier bn_attn_prefill_bf16) for the same S, theta, position_offset;
 *   then call bn_attn_prefill_bf16(q_out, NULL, v_out, ..., flags = BN_PREFILL_REUSE_ROTATED_K).
 *   pool / page_table (may be NULL): rotated K and V of token s of sequence b are also written to position
 *   s + position_offset of that sequence's pages (row b of page_table).
 * D must be 64; hidden a multiple of 8. */
BN_API int bn_attn_prefill_bf16_table(int B, int S, int Hkv, int D, float theta, int position_offset, void* workspace,
                                      size_t workspace_bytes, bn_stream_t stream);
BN_API int bn_gemm_qkv_rope_bf16(const void* x, const void* wqkv_t, void* q_out, void* v_out, int B, int S, int hidden,
                                 int Hq, int Hkv, int D, int position_offset, void* prefill_workspace,
                                 size_t prefill_workspace_bytes, void* pool, int64_t pool_pages,
                                 const int32_t* page_table, int max_pages, int* error_word, bn_stream_t stream);

/* Paged KV cache.  One pool per layer:
 *   pool[page][kv_head][0=K,1=V][BN_PAGE_TOKENS][D]  bf16
 * K is stored rotated (RoPE at the token's position), V as is.
 * page_table (n_seqs, max_pages) int32 maps a sequence's logical page to a
 * pool page.
 *
 * bn_kv_append: for t in [0,T): token of sequence seq_ids[t] at position
 * positions[t]; k_new, v_new (T, Hkv*D) with row stride in elements; dtype 0 =
 * fp32, 1 = bf16.  Fuses RoPE(K) (src/ops/op_rope.cuh:55-99), the bf16
 * conversion and the page write. */
BN_API int bn_kv_append(void* pool, int64_t pool_pages, const int32_t* page_table, int max_pages, const int32_t* seq_ids,
                 const int32_t* positions, int T, const void* k_new, const void* v_new, int64_t kv_row_stride,
                 int dtype, int Hkv, int D, float theta, bn_stream_t stream);

/* Bytes of scratch bn_attn_decode_paged needs (partial results of sequences
 * that span several SMs + tickets), for the same chunk_tokens.
 * The scratch must be zero-filled once before its first use; the kernel leaves
 * it clean for the next call.  The words that must stay clean (the tickets)
 * have a fixed place that depends on Hkv only, so one buffer sized for the
 * largest batch may serve calls with any smaller B, max_seq_len and
 * chunk_tokens, one call at a time, as long as Hkv is the same. */
BN_API size_t bn_attn_decode_workspace_bytes(int B, int Hq, int Hkv, int D, int max_seq_len, int chunk_tokens);

/* Single-token decode over the paged cache: for every sequence b the last row
 * of a per-head prefill over its seq_lens[b] cached tokens.
 *   q (B, Hq, D) bf16; rope_q != 0 rotates it in-kernel at position
 *   q_positions[b] (NULL: seq_lens[b]-1).
 *   out (B, Hq, D) bf16 (may be NULL); out_f32 (B, Hq, D) fp32 (may be NULL);
 *   lse (B, Hq) fp32 natural log (may be NULL; -inf for an empty sequence).
 * All cached tokens of the launch are cut into equal contiguous ranges, one per
 * SM, whatever the individual lengths; a (sequence, KV head) that falls into
 * several ranges is merged by a log-sum-exp combine inside the same launch.
 * chunk_tokens (0 = default 1024; else a multiple of 128) is the shortest range
 * an SM is given (fewer SMs take part when there is less work than that);
 * max_seq_len bounds seq_lens and sizes the scratch.  At most 1024 sequences
 * per launch. */
BN_API int bn_attn_decode_paged(const void* q, const void* pool, int64_t pool_pages, const int32_t* page_table,
                         int max_pages, const int32_t* seq_lens, const int32_t* q_positions, void* out,
                         float* out_f32, float* lse, int B, int Hq, int Hkv, int D, float scale, float theta,
                         int rope_q, int max_seq_len, int chunk_tokens, void* workspace, size_t workspace_bytes,
                         bn_stream_t stream);

/* The same decode for callers that cannot hand over a scratch buffer.
 * (No counterpart in the reference, which has neither a KV cache nor a decode operator.)
 *
 * Who needs it: code that runs where device allocation is off limits — a plugin called from inside someone else's
 * memory plan (a serving engine that has already carved up all of HBM, an inference graph whose buffers were fixed
 * at load time), or a real-time loop that may not touch the allocator because cudaMalloc/cudaFree synchronise the
 * device.  Such a caller still owns q, the cache and the outputs, but has nowhere to put the split-KV partials.
 *
 * Here the partials live in an array built into the library's device image (about 3.3 MB, held by every GPU that
 * loads the library until the process exits).  The call makes no cudaMalloc / cudaFree and calls no allocating
 * routine.  Limits: B * Hkv <= 256 and max_seq_len <= 4096; anything larger returns BN_ERR_UNSUPPORTED and
 * belongs to bn_attn_decode_paged.  Arguments as bn_attn_decode_paged, minus chunk_tokens and the workspace.
 *
 * The first call on each device looks up the array's device address and clears its header with that device
 * current; make that first call outside any stream capture.  All calls on a device share the one array, which
 * keeps what the previous call left (the kernel re-arms its own counters, which sit at a fixed place whatever the
 * batch size): calls that overlap on the GPU — two streams, two host threads — race on it; issue them on one
 * stream or otherwise serialise them. */
BN_API int bn_attn_decode_paged_static(const void* q, const void* pool, int64_t pool_pages, const int32_t* page_table,
                                       int max_pages, const int32_t* seq_lens, const int32_t* q_positions, void* out,
                                       float* out_f32, float* lse, int B, int Hq, int Hkv, int D, float scale,
                                       float theta, int rope_q, int max_seq_len, bn_stream_t stream);

/* bn_workspace_status for the built-in scratch of bn_attn_decode_paged_static, whose address the caller does not
 * have (no counterpart in the reference).  Waits for `stream`, reads the scratch's error word and returns BN_OK,
 * or BN_ERR_TIMEOUT when a call gave up on a bounded wait; in that case the header and the counters are cleared
 * here, so the next call starts clean.  Allocates nothing; it synchronises, so keep it off the hot path. */
BN_API int bn_attn_decode_paged_static_status(bn_stream_t stream);

/* Log-sum-exp merge of P partial attention results (split-KV across GPUs):
 *   outs (P, n, D) fp32 normalised partial outputs, lses (P, n) natural log
 *   (-inf = empty part)  ->  out_f32 (n, D) and/or out_bf16 (n, D), lse (n). */
BN_API int bn_attn_lse_combine(const float* outs, const float* lses, int P, int64_t n, int D, float* out_f32,
                        void* out_bf16, float* lse, bn_stream_t stream);

/* Same merge with explicit strides (in floats) between the parts of `outs` and
 * of `lses`, so that the P parts may sit in one gathered buffer per rank,
 * e.g. [n*D outputs | n log-sum-exps] repeated P times (what one all-gather of
 * each rank's contiguous send buffer produces). */
BN_API int bn_attn_lse_combine_strided(const float* outs, int64_t outs_part_stride, const float* lses,
                                       int64_t lses_part_stride, int P, int64_t n, int D, float* out_f32,
                                       void* out_bf16, float* lse, bn_stream_t stream);

/* ------------------------------------------------------------------------
 * Exchange + merge over peer memory (sequence split across the GPUs of a node)
 * ------------------------------------------------------------------------
 * The merge of bn_attn_lse_combine with the exchange in the same launch: every rank stores its partial (n rows of D
 * outputs, then n log-sum-exps: the layout the decode kernel writes when out_f32 and lse point into one buffer)
 * into every rank's exchange buffer with plain peer stores - every value with the step number beside it, so no fence
 * and no separate flag is needed - and merges in rank order, reading each rank's values again (bounded) until this
 * step's number stands beside them, so all ranks end with identical results.  No counterpart in the reference,
 * which is single-GPU.
 *
 *   bn_exchange_create       one per rank (allocates the buffer: 2 * world * n * (D + 1) * 8 bytes + 512 bytes);
 *   bn_exchange_ipc_handle   64 bytes that name the buffer to the other processes of the node; the caller gathers
 *                            the handles of all ranks (rank order) with whatever transport it has;
 *   bn_exchange_open_peers   maps the other ranks' buffers (handles = world * 64 bytes); loopback != 0 instead keeps
 *                            everything in this process (world 1, or a test that lets a wait run out);
 *   bn_exchange_combine      one launch per step on every rank, in the same order on all of them; wait_us bounds the
 *                            wait for the slowest rank (0 = one second); the step count is kept in the buffer, so
 *                            the launch may be captured into a CUDA graph and replayed;
 *   bn_exchange_status       synchronises `stream`; BN_ERR_TIMEOUT if a wait ran out (the exchange must then be
 *                            destroyed: the ranks are out of step);
 *   bn_exchange_destroy      unmaps and frees.
 * n * (D + 1) must be a multiple of 4; world <= 16. */
typedef struct bn_exchange bn_exchange_t;
BN_API int bn_exchange_create(int n, int D, int world, int rank, bn_exchange_t** out);
BN_API int bn_exchange_ipc_handle(bn_exchange_t* x, void* handle64);
BN_API int bn_exchange_open_peers(bn_exchange_t* x, const void* handles, int loopback);
BN_API int bn_exchange_combine(bn_exchange_t* x, const float* partial, float* out, float* lse, unsigned wait_us,
                               bn_stream_t stream);
BN_API int bn_exchange_status(bn_exchange_t* x, bn_stream_t stream);
BN_API void bn_exchange_destroy(bn_exchange_t* x);

#ifdef __cplusplus
}
#endif
#endif /* BN_ATTN_H_ */

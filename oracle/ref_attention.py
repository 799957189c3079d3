"""CPU restatement (numpy) of BareNet's grouped-query attention math.

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA path: it is
imported by the test-suite, by the smoke entry and by the CPU-baseline leg of
the benchmark, and by nothing that ships.  The product never falls back to it.

Parity status: the reference carries no golden vectors or numeric assertions
for this path (its test script prints shapes only), so this restatement is
pinned against outputs of the reference's own CUDA operators executed on a
B200 (see tests/golden/README.md for the generating recipe and files).

Each function names the reference source it restates (paths are relative to
the reference project root).
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


# ----------------------------------------------------------------------------
# bf16 helpers (numpy has no bfloat16; values are carried as float32 that are
# exactly representable in bf16, bit patterns as uint16)
# ----------------------------------------------------------------------------
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit pattern (uint16)."""
    x = np.ascontiguousarray(x, dtype=F32)
    u = x.view(np.uint32).astype(np.uint64)
    rounding = ((u >> 16) & 1) + 0x7FFF
    out = ((u + rounding) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        out[nan] = 0x7FC0
    return out


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(F32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """float32 values rounded to the nearest bf16, returned as float32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# ----------------------------------------------------------------------------
# RoPE   (src/ops/op_rope.cuh:55-99, launcher :101-126)
# ----------------------------------------------------------------------------
def rope_inv_freq(head_dim: int, theta: float = 10000.0) -> np.ndarray:
    """freq_i = 1.0 / powf(theta, float(2 i) / head_dim), i in [0, head_dim/2).

    src/ops/op_rope.cuh:82 — the exponent is formed in fp32, powf is the fp32
    power, the reciprocal is taken in double and rounded back to fp32.
    (glibc's powf and CUDA's powf can differ in the last bit; tests that need
    bit-identical angles pass the device-dumped table in through `inv_freq`.)
    """
    i2 = (2 * np.arange(head_dim // 2)).astype(F32)
    expo = i2 / F32(head_dim)
    # fp32 power, evaluated in double and rounded (numpy's own float32 pow is a
    # few ulp off; glibc's powf is correctly rounded on these arguments)
    p = np.power(np.float64(F32(theta)), expo.astype(np.float64)).astype(F32)
    return (1.0 / p.astype(np.float64)).astype(F32)


def rope_cos_sin(positions: np.ndarray, head_dim: int, theta: float = 10000.0,
                 inv_freq: np.ndarray | None = None):
    """cos/sin of angle = float(position) * freq, everything in fp32.

    src/ops/op_rope.cuh:79-86.
    """
    if inv_freq is None:
        inv_freq = rope_inv_freq(head_dim, theta)
    pos = np.asarray(positions).astype(F32)
    ang = (pos[:, None] * inv_freq[None, :].astype(F32)).astype(F32)
    return np.cos(ang, dtype=F32), np.sin(ang, dtype=F32)


def rope(x: np.ndarray, position_offset: int = 0, head_dim: int = 64,
         theta: float = 10000.0, positions: np.ndarray | None = None,
         inv_freq: np.ndarray | None = None, dtype=F32) -> np.ndarray:
    """Adjacent-pair rotary embedding applied independently to every
    head_dim-wide column block of a (rows, cols) matrix.

    src/ops/op_rope.cuh:55-99:  y[2i] = x[2i] c - x[2i+1] s ;
                                y[2i+1] = x[2i] s + x[2i+1] c
    with row r at position r + position_offset.  `dtype` float64 evaluates the
    rotation in double on the same fp32 angles (used as the exact reference
    for the bf16 path).
    """
    rows, cols = x.shape
    assert cols % head_dim == 0
    if positions is None:
        positions = np.arange(rows) + position_offset
    c, s = rope_cos_sin(positions, head_dim, theta, inv_freq)
    c = c.astype(dtype)
    s = s.astype(dtype)
    xv = x.astype(dtype).reshape(rows, cols // head_dim, head_dim // 2, 2)
    x0 = xv[..., 0]
    x1 = xv[..., 1]
    y = np.empty_like(xv)
    y[..., 0] = x0 * c[:, None, :] - x1 * s[:, None, :]
    y[..., 1] = x0 * s[:, None, :] + x1 * c[:, None, :]
    return y.reshape(rows, cols)


# ----------------------------------------------------------------------------
# KV head repeat  (mygrad/llama/llama_layers.py:105-138,
#                  src/llama/llama_layers.hpp:131-175)
# ----------------------------------------------------------------------------
def repeat_kv(kv: np.ndarray, n_rep: int, head_dim: int) -> np.ndarray:
    """dst head kv_head*n_rep+rep  <-  src head kv_head."""
    if n_rep == 1:
        return kv
    rows, w = kv.shape
    n_kv = w // head_dim
    return np.repeat(kv.reshape(rows, n_kv, 1, head_dim), n_rep, axis=2).reshape(rows, n_kv * n_rep * head_dim)


# ----------------------------------------------------------------------------
# softmax  (src/ops/op_softmax.cuh:76-151 causal, :8-72 plain)
# ----------------------------------------------------------------------------
def softmax_rows(scores: np.ndarray, causal: bool, seq_offset: int = 0, dtype=F32) -> np.ndarray:
    """Row softmax; with `causal`, column j of row r is valid iff
    j <= r + seq_offset, masked entries become exactly 0."""
    s = scores.astype(dtype)
    rows, cols = s.shape
    if causal:
        valid = np.arange(cols)[None, :] <= (np.arange(rows)[:, None] + seq_offset)
    else:
        valid = np.ones((rows, cols), dtype=bool)
    neg = np.where(valid, s, -np.inf)
    m = neg.max(axis=1, keepdims=True)
    e = np.where(valid, np.exp((s - m).astype(dtype)), 0).astype(dtype)
    return (e / e.sum(axis=1, keepdims=True, dtype=dtype)).astype(dtype)


# ----------------------------------------------------------------------------
# The attention core in the reference's own ("collapsed") semantics
# (mygrad/llama/llama_layers.py:161-183; C++ mirror
#  src/llama/llama_layers.hpp:82-109)
# ----------------------------------------------------------------------------
def attention_collapsed(q: np.ndarray, k: np.ndarray, v: np.ndarray, *, num_heads: int,
                        num_kv_heads: int, head_dim: int, theta: float = 10000.0,
                        position_offset: int = 0, causal: bool = True, dtype=F32,
                        inv_freq=None, apply_rope: bool = True) -> np.ndarray:
    """q (S, Hq*D), k,v (S, Hkv*D) pre-RoPE  ->  (S, Hq*D).

    The reference never splits heads (llama_layers.py:87-103 is a no-op): the
    score matrix is ONE (S,S) product over the full Hq*D width, one softmax,
    one P@V with V repeated per query head.
    """
    scale = dtype(1.0 / np.sqrt(head_dim))
    if apply_rope:
        q = rope(q, position_offset, head_dim, theta, inv_freq=inv_freq, dtype=dtype)
        k = rope(k, position_offset, head_dim, theta, inv_freq=inv_freq, dtype=dtype)
    n_rep = num_heads // num_kv_heads
    kr = repeat_kv(k.astype(dtype), n_rep, head_dim)
    vr = repeat_kv(v.astype(dtype), n_rep, head_dim)
    scores = (q.astype(dtype) @ kr.T).astype(dtype) * scale
    p = softmax_rows(scores, causal, position_offset, dtype)
    return (p @ vr).astype(dtype)


def gqa_layer_collapsed(x, wq, wk, wv, wo, *, num_heads, num_kv_heads, head_dim,
                        theta=10000.0, position_offset=0, causal=True, dtype=F32, inv_freq=None):
    """Whole GroupedQueryAttention.__call__ (mygrad/llama/llama_layers.py:140-188):
    x (S, hidden); weights stored (in, out)."""
    x = x.astype(dtype)
    q = x @ wq.astype(dtype)
    k = x @ wk.astype(dtype)
    v = x @ wv.astype(dtype)
    a = attention_collapsed(q, k, v, num_heads=num_heads, num_kv_heads=num_kv_heads,
                            head_dim=head_dim, theta=theta, position_offset=position_offset,
                            causal=causal, dtype=dtype, inv_freq=inv_freq)
    return (a @ wo.astype(dtype)).astype(dtype)


# ----------------------------------------------------------------------------
# Per-head grouped-query attention: the same operators applied independently
# to every head_dim-wide head, query head h reading KV head h // n_rep
# (head map: mygrad/llama/llama_layers.py:126-136).
# ----------------------------------------------------------------------------
def attention_per_head(q: np.ndarray, k: np.ndarray, v: np.ndarray, *, num_heads: int,
                       num_kv_heads: int, head_dim: int, theta: float = 10000.0,
                       position_offset: int = 0, causal: bool = True, dtype=np.float64,
                       inv_freq=None, apply_rope: bool = True, round_rope_bf16: bool = False,
                       return_lse: bool = False):
    """q (S, Hq*D), k,v (S, Hkv*D).  The reference's position rule: row r of q
    AND of k sits at position r + position_offset (llama_layers.py:162-163) and
    key j is valid iff j <= r + position_offset (src/ops/op_softmax.cuh:88-101).
    `round_rope_bf16` rounds the rotated Q/K to bf16 (what a bf16 tensor-core
    path feeds its MMAs)."""
    S = q.shape[0]
    assert k.shape[0] == S and v.shape[0] == S
    scale = 1.0 / np.sqrt(head_dim)
    if apply_rope:
        q = rope(q, position_offset, head_dim, theta, inv_freq=inv_freq, dtype=dtype)
        k = rope(k, position_offset, head_dim, theta, inv_freq=inv_freq, dtype=dtype)
        if round_rope_bf16:
            q = round_bf16(q.astype(F32)).astype(dtype)
            k = round_bf16(k.astype(F32)).astype(dtype)
    q = q.astype(dtype).reshape(S, num_heads, head_dim)
    k = k.astype(dtype).reshape(S, num_kv_heads, head_dim)
    v = v.astype(dtype).reshape(S, num_kv_heads, head_dim)
    n_rep = num_heads // num_kv_heads
    out = np.empty((S, num_heads, head_dim), dtype=dtype)
    lse = np.empty((S, num_heads), dtype=dtype)
    valid = (np.arange(S)[None, :] <= np.arange(S)[:, None] + position_offset) if causal else np.ones((S, S), dtype=bool)
    for h in range(num_heads):
        g = h // n_rep
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = np.where(valid, s, -np.inf)
        m = s.max(axis=1, keepdims=True)
        e = np.exp(s - m)
        l = e.sum(axis=1, keepdims=True)
        out[:, h, :] = (e / l) @ v[:, g, :]
        lse[:, h] = (m + np.log(l))[:, 0]
    out = out.reshape(S, num_heads * head_dim)
    return (out, lse) if return_lse else out


# ----------------------------------------------------------------------------
# Paged single-token decode.  The reference has no KV cache
# (mygrad/llama/llama_model.py:136-144 recomputes the whole sequence and takes
# the last row), so the definition of decode is: the last row of a full
# per-head prefill over the cached keys/values.
# ----------------------------------------------------------------------------
PAGE_TOKENS = 16


def paged_gather(pool: np.ndarray, page_table_row: np.ndarray, length: int):
    """pool: (num_pages, Hkv, 2, PAGE_TOKENS, D) values.  Returns K, V of shape
    (length, Hkv, D) in token order."""
    n_pages = (length + PAGE_TOKENS - 1) // PAGE_TOKENS
    pages = pool[page_table_row[:n_pages]]            # (n_pages, Hkv, 2, 16, D)
    k = pages[:, :, 0].transpose(0, 2, 1, 3).reshape(n_pages * PAGE_TOKENS, pool.shape[1], pool.shape[-1])
    v = pages[:, :, 1].transpose(0, 2, 1, 3).reshape(n_pages * PAGE_TOKENS, pool.shape[1], pool.shape[-1])
    return k[:length], v[:length]


def decode_paged(q: np.ndarray, pool: np.ndarray, page_table: np.ndarray, seq_lens: np.ndarray, *,
                 num_heads: int, num_kv_heads: int, head_dim: int, theta: float = 10000.0,
                 rope_q: bool = True, dtype=np.float64, inv_freq=None, return_lse: bool = False,
                 token_begin: np.ndarray | None = None, token_end: np.ndarray | None = None):
    """q (B, Hq*D) pre-RoPE (position = seq_len-1 of its sequence); cache holds
    post-RoPE K and V.  Returns (B, Hq*D) [and lse (B, Hq)].

    token_begin/token_end restrict each sequence to a token sub-range (what a
    sequence-parallel shard holds); an empty range yields out=0, lse=-inf.
    """
    B = q.shape[0]
    out = np.zeros((B, num_heads * head_dim), dtype=dtype)
    lse = np.full((B, num_heads), -np.inf, dtype=dtype)
    n_rep = num_heads // num_kv_heads
    scale = 1.0 / np.sqrt(head_dim)
    for b in range(B):
        L = int(seq_lens[b])
        if L == 0:
            continue
        qb = q[b:b + 1].astype(F32)
        if rope_q:
            qb = rope(qb, head_dim=head_dim, theta=theta, positions=np.array([L - 1]),
                      inv_freq=inv_freq, dtype=dtype)
            qb = round_bf16(qb.astype(F32))
        qb = qb.astype(dtype).reshape(num_heads, head_dim)
        k, v = paged_gather(pool, page_table[b], L)
        t0 = 0 if token_begin is None else int(token_begin[b])
        t1 = L if token_end is None else min(L, int(token_end[b]))
        if t1 <= t0:
            continue
        k = k[t0:t1].astype(dtype)
        v = v[t0:t1].astype(dtype)
        for h in range(num_heads):
            g = h // n_rep
            s = (k[:, g, :] @ qb[h]) * scale
            m = s.max()
            e = np.exp(s - m)
            l = e.sum()
            out[b, h * head_dim:(h + 1) * head_dim] = (e / l) @ v[:, g, :]
            lse[b, h] = m + np.log(l)
    return (out, lse) if return_lse else out


# ----------------------------------------------------------------------------
# Log-sum-exp merge of split-KV partials
# ----------------------------------------------------------------------------
def lse_combine(outs: np.ndarray, lses: np.ndarray, dtype=np.float64):
    """outs (P, ..., D) normalised partial outputs, lses (P, ...) natural-log
    sum-exp of each part (-inf for an empty part).  Returns merged (..., D), (...)."""
    outs = outs.astype(dtype)
    lses = lses.astype(dtype)
    m = lses.max(axis=0)
    safe_m = np.where(np.isfinite(m), m, 0.0)
    w = np.exp(lses - safe_m[None])
    w = np.where(np.isfinite(lses), w, 0.0)
    tot = w.sum(axis=0)
    o = (outs * w[..., None]).sum(axis=0) / np.where(tot > 0, tot, 1.0)[..., None]
    lse = np.where(tot > 0, safe_m + np.log(np.where(tot > 0, tot, 1.0)), -np.inf)
    return o, lse


# ----------------------------------------------------------------------------
# Fused RoPE(K) + bf16 + page write (the step that fills the cache)
# ----------------------------------------------------------------------------
def kv_append(pool_bits: np.ndarray, page_table: np.ndarray, positions: np.ndarray, seq_ids: np.ndarray,
              k_new: np.ndarray, v_new: np.ndarray, *, head_dim: int, theta: float = 10000.0, inv_freq=None):
    """Writes token t (sequence seq_ids[t], position positions[t]) into the
    bf16 bit-pattern pool (num_pages, Hkv, 2, 16, D): K rotated at its position
    in fp32 (src/ops/op_rope.cuh:55-99) then rounded to bf16, V rounded."""
    T = k_new.shape[0]
    n_kv = pool_bits.shape[1]
    for t in range(T):
        pos = int(positions[t])
        page = int(page_table[int(seq_ids[t]), pos // PAGE_TOKENS])
        slot = pos % PAGE_TOKENS
        kr = rope(k_new[t:t + 1].astype(F32), head_dim=head_dim, theta=theta, positions=np.array([pos]),
                  inv_freq=inv_freq, dtype=F32)
        pool_bits[page, :, 0, slot, :] = f32_to_bf16_bits(kr.reshape(n_kv, head_dim))
        pool_bits[page, :, 1, slot, :] = f32_to_bf16_bits(v_new[t].astype(F32).reshape(n_kv, head_dim))
    return pool_bits


def rmsnorm(x: np.ndarray, weight: np.ndarray, eps: float = 1e-6, residual: np.ndarray | None = None,
            dtype=np.float64):
    """RMSNorm, row-wise: y = x / sqrt(mean(x^2) + eps) * w  (op_rmsnorm_kernel,
    src/ops/op_rmsnorm.cuh:8-53; `RMSNorm.__call__`, mygrad/llama/llama_layers.py:13-29).
    With `residual`, x + residual is normalised (the decoder layer's residual add followed by the next norm,
    llama_layers.py:279-283) and (sum, y) is returned.  This numpy form is the exact-math statement (float64 by
    default); the bit-faithful fp32 order of the reference kernel lives in oracle/ref_attention.c."""
    x = np.asarray(x, dtype=dtype)
    w = np.asarray(weight, dtype=dtype).reshape(1, -1)
    s = x if residual is None else (np.asarray(x, dtype=F32) + np.asarray(residual, dtype=F32)).astype(dtype)
    rms = np.sqrt((s * s).mean(axis=1, keepdims=True) + dtype(eps))
    y = s / rms * w
    return y if residual is None else (s, y)


def argmax_rows(x: np.ndarray) -> np.ndarray:
    """Per-row argmax with the reference's sequential rule: op_argmax (src/ops/op_reduction.cuh:196-210) runs
    MaxAccumFunc (:5-19) over the columns of a row in order -- accum starts as element 0 and is replaced only by a
    strictly greater value, so ties keep the first index and a NaN wins only at index 0.  Returns (rows, 1) uint32
    like TensorF.argmax (src/py_tensor_shim.hh:220-224)."""
    x = np.asarray(x, dtype=F32)
    out = np.zeros((x.shape[0], 1), dtype=np.uint32)
    for r in range(x.shape[0]):
        acc, ind = x[r, 0], 0
        for c in range(1, x.shape[1]):
            if x[r, c] > acc:
                acc, ind = x[r, c], c
        out[r, 0] = ind
    return out


def embed(table: np.ndarray, input_ids: np.ndarray) -> np.ndarray:
    """LLaMAModel.embed (mygrad/llama/llama_model.py:58-78): row i of the result is row input_ids[i] of the
    embedding table (the reference gathers on the host and uploads)."""
    table = np.asarray(table, dtype=F32)
    out = np.zeros((len(input_ids), table.shape[1]), dtype=F32)
    for i, token_id in enumerate(input_ids):
        out[i] = table[int(token_id)]
    return out

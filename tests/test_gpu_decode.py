"""Paged single-token decode, KV append and the LSE combine vs the oracle,
through the C ABI.  Gate: max abs err <= 2e-2 (bf16 inputs, fp32 accumulation)."""
import numpy as np
import pytest
import torch

from oracle import ref_attention as R

pytestmark = pytest.mark.gpu

GATE = 2e-2
Hq, Hkv, D = 32, 4, 64


def build_cache(lens, seed, extra_pages=3, poison=False):
    """Random cache contents with a permuted (non-contiguous) page table."""
    from baranet_bdml_b200.kv_cache import PagedKVCache, PAGE_TOKENS
    rng = np.random.default_rng(seed)
    B = len(lens)
    pages_per = [(L + PAGE_TOKENS - 1) // PAGE_TOKENS for L in lens]
    max_pages = max(max(pages_per), 1)
    n_pages = sum(pages_per) + extra_pages
    cache = PagedKVCache(n_pages, B, max_pages, Hkv, D)
    pool = R.round_bf16(rng.standard_normal((n_pages, Hkv, 2, PAGE_TOKENS, D), dtype=np.float32))
    perm = rng.permutation(n_pages)
    pt = np.zeros((B, max_pages), dtype=np.int32)
    at = 0
    for b in range(B):
        pt[b, :pages_per[b]] = perm[at:at + pages_per[b]]
        at += pages_per[b]
    if poison:
        # tokens past the end of a sequence's last page hold NaN/Inf: they must never reach the output
        for b, L in enumerate(lens):
            if L % PAGE_TOKENS:
                pool[pt[b, pages_per[b] - 1], :, :, L % PAGE_TOKENS:, :] = np.nan
    cache.pool.copy_(torch.from_numpy(pool).to(torch.bfloat16))
    cache.page_table.copy_(torch.from_numpy(pt))
    cache.seq_lens.copy_(torch.tensor(lens, dtype=torch.int32))
    q = R.round_bf16(rng.standard_normal((B, Hq * D), dtype=np.float32))
    return cache, pool, pt, q


def run_decode(cache, q, **kw):
    B = q.shape[0]
    tq = torch.from_numpy(q).cuda().to(torch.bfloat16).reshape(B, Hq, D)
    out32 = torch.empty((B, Hq, D), dtype=torch.float32, device="cuda")
    lse = torch.empty((B, Hq), dtype=torch.float32, device="cuda")
    out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device="cuda")
    cache.decode(tq, num_heads=Hq, out=out, out_f32=out32, lse=lse, **kw)
    torch.cuda.synchronize()
    cache.status()
    return out.float().cpu().numpy().reshape(B, -1), out32.cpu().numpy().reshape(B, -1), lse.cpu().numpy()


@pytest.mark.parametrize("lens", [[1], [16], [17], [1024], [4096], [5, 130, 16, 511, 512, 513, 2049],
                                  [0, 3, 0, 700],
                                  # no sequence above 2048 tokens and at least 16 (sequence, KV head) segments: CTAs take
                                  # whole segments (ragged, with empty sequences; more segments than CTAs in the last one)
                                  [5, 130, 16, 511, 512, 513, 2048, 1, 0, 257],
                                  [(37 * i) % 600 for i in range(50)]])
def test_decode_vs_oracle(lib, lens):
    cache, pool, pt, q = build_cache(lens, sum(lens) + len(lens), poison=True)
    got, got32, lse = run_decode(cache, q, max_seq_len=max(max(lens), 1))
    ref, ref_lse = R.decode_paged(q, np.nan_to_num(pool), pt, np.array(lens), num_heads=Hq, num_kv_heads=Hkv,
                                  head_dim=D, return_lse=True)
    assert np.isfinite(got32).all()
    assert np.abs(got32 - ref).max() <= GATE, np.abs(got32 - ref).max()
    assert np.abs(got - ref).max() <= GATE
    fin = np.isfinite(ref_lse)
    assert np.array_equal(np.isfinite(lse), fin)
    assert np.abs(lse[fin] - ref_lse[fin]).max() <= 2e-2


def test_decode_is_last_row_of_prefill(lib):
    """decode(t) == row t of a full prefill: K/V appended through bn_kv_append (RoPE fused)."""
    from baranet_bdml_b200.kv_cache import PagedKVCache
    rng = np.random.default_rng(11)
    S = 200
    qa = R.round_bf16(rng.standard_normal((S, Hq * D), dtype=np.float32))
    ka = R.round_bf16(rng.standard_normal((S, Hkv * D), dtype=np.float32))
    va = R.round_bf16(rng.standard_normal((S, Hkv * D), dtype=np.float32))
    ref = R.attention_per_head(qa, ka, va, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, dtype=np.float64,
                               round_rope_bf16=True)
    cache = PagedKVCache(40, 1, 13, Hkv, D)
    cache.page_table.copy_(torch.from_numpy(rng.permutation(40)[:13].astype(np.int32))[None])
    cache.append(torch.zeros(S, dtype=torch.int32, device="cuda"), torch.arange(S, dtype=torch.int32, device="cuda"),
                 torch.from_numpy(ka).cuda(), torch.from_numpy(va).cuda())
    for t in (0, 15, 16, 127, 199):
        cache.seq_lens.fill_(t + 1)
        got, got32, _ = run_decode(cache, qa[t:t + 1], max_seq_len=208)
        assert np.abs(got32[0] - ref[t]).max() <= GATE, (t, np.abs(got32[0] - ref[t]).max())


def test_kv_append_matches_oracle(lib):
    from baranet_bdml_b200.kv_cache import PagedKVCache
    rng = np.random.default_rng(12)
    T_ = 37
    cache = PagedKVCache(16, 3, 4, Hkv, D)
    pt = rng.permutation(16)[:12].astype(np.int32).reshape(3, 4)
    cache.page_table.copy_(torch.from_numpy(pt))
    seq = rng.integers(0, 3, T_).astype(np.int32)
    pos = np.array([rng.integers(0, 64) for _ in range(T_)], dtype=np.int32)
    # unique (seq,pos) pairs so the write order does not matter
    _, keep = np.unique(seq.astype(np.int64) * 1000 + pos, return_index=True)
    seq, pos = seq[keep], pos[keep]
    k = rng.standard_normal((len(seq), Hkv * D), dtype=np.float32)
    v = rng.standard_normal((len(seq), Hkv * D), dtype=np.float32)
    cache.append(torch.from_numpy(seq).cuda(), torch.from_numpy(pos).cuda(), torch.from_numpy(k).cuda(),
                 torch.from_numpy(v).cuda())
    torch.cuda.synchronize()
    got = cache.pool.view(torch.int16).cpu().numpy().view(np.uint16)
    ref = R.kv_append(np.zeros_like(got), pt, pos, seq, k, v, head_dim=D)
    # V is a pure bf16 rounding: bit exact.  K goes through cosf/sinf: allow 1 bf16 ulp.
    assert np.array_equal(got[:, :, 1], ref[:, :, 1])
    dk = np.abs(R.bf16_bits_to_f32(got[:, :, 0]) - R.bf16_bits_to_f32(ref[:, :, 0]))
    assert dk.max() <= 2.0 ** -6


@pytest.mark.parametrize("chunk", [128, 256, 1024, 8192])
def test_split_kv_chunks_agree(lib, chunk):
    lens = [3000, 777, 4096, 129]
    cache, pool, pt, q = build_cache(lens, 21)
    base, base32, base_lse = run_decode(cache, q, max_seq_len=4096, chunk_tokens=8192)
    got, got32, lse = run_decode(cache, q, max_seq_len=4096, chunk_tokens=chunk)
    assert np.abs(got32 - base32).max() <= 1e-3
    assert np.abs(lse - base_lse).max() <= 1e-3


def test_decode_twice_same_workspace(lib):
    """The scratch buffer is left clean: a second launch on it gives the same bits."""
    cache, pool, pt, q = build_cache([2000, 1500, 3000], 5)
    a = run_decode(cache, q, max_seq_len=3008, chunk_tokens=256)
    b = run_decode(cache, q, max_seq_len=3008, chunk_tokens=256)
    assert np.array_equal(a[1], b[1])


def test_config3_shape(lib, cref):
    """BASELINE config 3: batch 64, lengths uniform in [1024, 4096], 16-token pages."""
    rng = np.random.default_rng(3)
    lens = rng.integers(1024, 4097, 64).tolist()
    cache, pool, pt, q = build_cache(lens, 33)
    got, got32, lse = run_decode(cache, q, max_seq_len=max(lens), rope_q=False)
    ref, ref_lse = cref.decode_paged(q, R.f32_to_bf16_bits(pool), pt, np.array(lens, dtype=np.int32), num_heads=Hq,
                                     num_kv_heads=Hkv, head_dim=D)
    assert np.abs(got32 - ref).max() <= GATE
    assert np.abs(lse - ref_lse).max() <= 2e-2


def test_sequence_split_partials_combine(lib):
    """Long-context path on one GPU: the sequence cut into P token ranges (as P GPUs would hold
    them), one decode per range, partials merged by bn_attn_lse_combine == decode over the whole."""
    from baranet_bdml_b200 import ops
    from baranet_bdml_b200.kv_cache import PagedKVCache, PAGE_TOKENS
    L, P = 8192, 4
    cache, pool, pt, q = build_cache([L, L], 44)
    full, full32, full_lse = run_decode(cache, q, max_seq_len=L)
    outs, lses = [], []
    per = L // P
    qpos = torch.full((2,), L - 1, dtype=torch.int32, device="cuda")
    tq = torch.from_numpy(q).cuda().to(torch.bfloat16).reshape(2, Hq, D)
    for r in range(P):
        sub_pt = cache.page_table[:, r * per // PAGE_TOKENS:(r + 1) * per // PAGE_TOKENS].contiguous()
        sl = torch.full((2,), per, dtype=torch.int32, device="cuda")
        o = torch.empty((2, Hq, D), dtype=torch.float32, device="cuda")
        l = torch.empty((2, Hq), dtype=torch.float32, device="cuda")
        cache.decode(tq, num_heads=Hq, out_f32=o, lse=l, q_positions=qpos, seq_lens=sl, page_table=sub_pt,
                     max_seq_len=per)
        outs.append(o.reshape(2 * Hq, D))
        lses.append(l.reshape(2 * Hq))
    merged, mlse = ops.lse_combine(torch.stack(outs), torch.stack(lses))
    torch.cuda.synchronize()
    assert np.abs(merged.cpu().numpy().reshape(2, -1) - full32).max() <= 1e-3
    assert np.abs(mlse.cpu().numpy().reshape(2, -1) - full_lse).max() <= 1e-3


def test_lse_combine_edge_cases(lib):
    from baranet_bdml_b200 import ops
    rng = np.random.default_rng(8)
    P, n, Dd = 5, 7, 64
    outs = rng.standard_normal((P, n, Dd), dtype=np.float32)
    lses = rng.standard_normal((P, n)).astype(np.float32) * 5
    lses[1, :] = -np.inf          # an empty shard
    lses[:, 3] = -np.inf          # a row empty everywhere
    lses[2, 4] = 80.0             # one dominant shard
    got, glse = ops.lse_combine(torch.from_numpy(outs).cuda(), torch.from_numpy(lses).cuda())
    ref, rlse = R.lse_combine(outs, lses)
    assert np.abs(got.cpu().numpy() - ref).max() <= 1e-5
    g = glse.cpu().numpy()
    assert np.array_equal(np.isfinite(g), np.isfinite(rlse))
    assert np.abs(g[np.isfinite(g)] - rlse[np.isfinite(rlse)]).max() <= 1e-5
    assert np.abs(got.cpu().numpy()[4] - outs[2, 4]).max() <= 1e-6


def test_lse_combine_on_a_gathered_buffer(lib):
    """The layout one all-gather produces: per rank [n*D outputs | n log-sum-exps], P ranks back to back."""
    from baranet_bdml_b200 import _lib
    rng = np.random.default_rng(9)
    P, n, Dd = 4, 12, 64
    outs = rng.standard_normal((P, n, Dd), dtype=np.float32)
    lses = (rng.standard_normal((P, n)) * 3).astype(np.float32)
    lses[2, 5] = -np.inf
    buf = np.concatenate([np.concatenate([outs[r].reshape(-1), lses[r]]) for r in range(P)]).astype(np.float32)
    t = torch.from_numpy(buf).cuda()
    out = torch.empty((n, Dd), dtype=torch.float32, device="cuda")
    lse = torch.empty((n,), dtype=torch.float32, device="cuda")
    stride = n * (Dd + 1)
    _lib.check(lib.bn_attn_lse_combine_strided(t.data_ptr(), stride, t.data_ptr() + 4 * n * Dd, stride, P, n, Dd,
                                               out.data_ptr(), None, lse.data_ptr(), None))
    torch.cuda.synchronize()
    ref, rlse = R.lse_combine(outs, lses)
    assert np.abs(out.cpu().numpy() - ref).max() <= 1e-5
    assert np.abs(lse.cpu().numpy() - rlse).max() <= 1e-5


def test_partial_exchange_single_rank(lib):
    """PartialExchange without a process group: the merge of one part is the part itself."""
    from baranet_bdml_b200.dist import PartialExchange
    ex = PartialExchange(6, 64)
    ex.out_view.copy_(torch.arange(6 * 64, dtype=torch.float32, device="cuda").view(6, 64))
    ex.lse_view.copy_(torch.linspace(-2, 2, 6, device="cuda"))
    o, l = ex.combine()
    torch.cuda.synchronize()
    assert torch.equal(o, ex.out_view) and torch.allclose(l, ex.lse_view, atol=1e-6)

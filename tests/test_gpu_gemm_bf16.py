"""bf16 tcgen05 GEMM (C = A @ Bt^T, fp32 accumulation) through the C ABI against an fp64 product of the same
bf16-rounded operands.  Gate: max|got - ref| <= 2^-8 * max|ref| (one bf16 ulp at the largest magnitude) + the
accumulation-order slack of fp32, far below it."""
import numpy as np
import pytest
import torch

from oracle import ref_attention as R

pytestmark = pytest.mark.gpu


def run_case(M, N, K, seed):
    from baranet_bdml_b200 import ops
    rng = np.random.default_rng(seed)
    a = R.round_bf16(rng.standard_normal((M, K), dtype=np.float32))
    bt = R.round_bf16((rng.standard_normal((N, K)) * 0.05).astype(np.float32))
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = ops.gemm_bf16_nt(torch.from_numpy(a).cuda().to(torch.bfloat16), torch.from_numpy(bt).cuda().to(torch.bfloat16),
                           error_word=err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref = a.astype(np.float64) @ bt.astype(np.float64).T
    return got.float().cpu().numpy(), ref


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 2048), (256, 512, 128), (1, 8, 8), (100, 264, 72),
                                   (129, 257 // 8 * 8, 65 // 8 * 8), (300, 2048, 2048), (1000, 512, 2048),
                                   (4096, 256, 256)])
def test_gemm_matches_fp64_product(lib, M, N, K):
    got, ref = run_case(M, N, K, M + 3 * N + 7 * K)
    scale = max(np.abs(ref).max(), 1e-30)
    assert np.abs(got - ref).max() <= scale * 2.0 ** -8, (M, N, K, np.abs(got - ref).max() / scale)


def test_gemm_projection_shapes_of_the_layer(lib):
    """q_proj / k_proj of TinyLLaMA on 2048 tokens: (2048, 2048) @ (2048, 2048)^T and (2048, 2048) @ (256, 2048)^T;
    linearity in A: gemm(2a) == 2 gemm(a) exactly (a power-of-two scale commutes with every rounding)."""
    from baranet_bdml_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((2048, 2048), generator=g, device="cuda").to(torch.bfloat16)
    for n_out in (2048, 256):
        w = (torch.randn((n_out, 2048), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        y = ops.gemm_bf16_nt(x, w)
        y2 = ops.gemm_bf16_nt((x.float() * 2).to(torch.bfloat16), w)
        torch.cuda.synchronize()
        assert torch.equal(y2.float(), y.float() * 2)
        ref = x.double() @ w.double().T
        assert float((y.double() - ref).abs().max()) <= float(ref.abs().max()) * 2.0 ** -8


def test_gemm_rejects_bad_arguments(lib):
    from baranet_bdml_b200 import ops
    a = torch.zeros((16, 12), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="multiples of 8"):
        ops.gemm_bf16_nt(a, torch.zeros((8, 12), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(RuntimeError, match="inner dimensions mismatch"):
        ops.gemm_bf16_nt(torch.zeros((16, 16), dtype=torch.bfloat16, device="cuda"),
                         torch.zeros((8, 8), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(RuntimeError, match="only GPU implementation available"):
        ops.gemm_bf16_nt(torch.zeros((16, 16), dtype=torch.bfloat16), torch.zeros((8, 16), dtype=torch.bfloat16))


def test_bf16_layer_against_staged_fp64_restatement(lib):
    """The whole attention layer on the bf16 path (4 tcgen05 GEMMs + the fused attention core) against the oracle's
    per-head attention with fp64 arithmetic and a bf16 rounding wherever the kernels round (q, k, v, attention output,
    layer output).  Gate 2e-2 absolute, the bf16 tolerance of the path."""
    import torch
    from baranet_bdml_b200.layers import GroupedQueryAttentionBF16, LLaMAConfig
    cfg = LLaMAConfig(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, intermediate_size=1024,
                      num_hidden_layers=1)
    np.random.seed(5)
    layer = GroupedQueryAttentionBF16(cfg)
    B, S = 2, 300
    rng = np.random.default_rng(8)
    x = R.round_bf16(rng.standard_normal((B, S, cfg.hidden_size), dtype=np.float32))
    got = layer(torch.from_numpy(x).cuda().to(torch.bfloat16), position_offset=2).float().cpu().numpy()
    wq, wk, wv, wo = (w.float().cpu().numpy().astype(np.float64) for w in (layer.q_proj, layer.k_proj, layer.v_proj,
                                                                          layer.o_proj))
    for b in range(B):
        xb = x[b].astype(np.float64)
        q, k, v = (R.round_bf16((xb @ w.T).astype(np.float32)) for w in (wq, wk, wv))
        attn = R.attention_per_head(q, k, v, num_heads=8, num_kv_heads=2, head_dim=64, position_offset=2, causal=True,
                                    dtype=np.float64, round_rope_bf16=True)
        ref = R.round_bf16(attn.astype(np.float32)).astype(np.float64) @ wo.T
        assert np.abs(got[b] - ref).max() <= 2e-2, np.abs(got[b] - ref).max()


@pytest.mark.parametrize("M,inter,K", [(128, 128, 64), (200, 256, 128), (64, 5632, 2048), (300, 136, 72), (1000, 1000, 512)])
def test_swiglu_gemm_against_fp64(lib, M, inter, K):
    """silu(x Wg) * (x Wu) from one launch against fp64 on the same bf16 operands; the kernel applies the activation
    to its fp32 accumulators and rounds once, so the gate is one bf16 ulp at the largest magnitude."""
    from baranet_bdml_b200 import ops
    rng = np.random.default_rng(M + inter + K)
    x = R.round_bf16(rng.standard_normal((M, K), dtype=np.float32))
    wg = R.round_bf16((rng.standard_normal((inter, K)) * 0.05).astype(np.float32))
    wu = R.round_bf16((rng.standard_normal((inter, K)) * 0.05).astype(np.float32))
    tx, tg, tu = (torch.from_numpy(a).cuda().to(torch.bfloat16) for a in (x, wg, wu))
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = ops.gemm_swiglu_bf16_nt(tx, ops.pack_gate_up(tg, tu), inter, error_word=err).float().cpu().numpy()
    assert int(err.item()) == 0
    g = x.astype(np.float64) @ wg.astype(np.float64).T
    u = x.astype(np.float64) @ wu.astype(np.float64).T
    ref = g / (1.0 + np.exp(-g)) * u
    assert np.abs(got - ref).max() <= max(np.abs(ref).max(), 1e-30) * 2.0 ** -8


def test_bf16_mlp_against_staged_fp64(lib):
    """MLPBF16 (fused gate/up GEMM + down GEMM) against fp64 with a bf16 rounding of the intermediate, where the
    kernels round."""
    from baranet_bdml_b200.layers import LLaMAConfig, MLPBF16
    cfg = LLaMAConfig(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, intermediate_size=1408,
                      num_hidden_layers=1)
    np.random.seed(2)
    mlp = MLPBF16(cfg)
    rng = np.random.default_rng(4)
    x = R.round_bf16(rng.standard_normal((333, 512), dtype=np.float32))
    got = mlp(torch.from_numpy(x).cuda().to(torch.bfloat16)).float().cpu().numpy()
    wg, wu, wd = (w.float().cpu().numpy().astype(np.float64) for w in (mlp.gate_proj, mlp.up_proj, mlp.down_proj))
    g, u = x.astype(np.float64) @ wg.T, x.astype(np.float64) @ wu.T
    inter = R.round_bf16((g / (1.0 + np.exp(-g)) * u).astype(np.float32)).astype(np.float64)
    ref = inter @ wd.T
    assert np.abs(got - ref).max() <= np.abs(ref).max() * 2.0 ** -7


def test_bf16_decoder_layer_against_staged_fp64(lib):
    """The whole pre-norm decoder block on the bf16 path (norm, attention layer, fused residual add + norm, SwiGLU MLP,
    residual) against fp64 with a bf16 rounding wherever a kernel rounds; and two stacked layers with the deferred
    residual add (`forward_parts(pending=...)`) equal to the plain composition."""
    from baranet_bdml_b200.layers import LLaMAConfig, LLaMADecoderLayerBF16
    cfg = LLaMAConfig(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, intermediate_size=1408,
                      num_hidden_layers=2)
    np.random.seed(12)
    layer = LLaMADecoderLayerBF16(cfg)
    B, S, H = 2, 200, 512
    rng = np.random.default_rng(3)
    x = R.round_bf16(rng.standard_normal((B, S, H), dtype=np.float32))
    tx = torch.from_numpy(x).cuda().to(torch.bfloat16)
    got = layer(tx).float().cpu().numpy()

    rb = lambda a: R.round_bf16(np.asarray(a, dtype=np.float32)).astype(np.float64)
    f64 = lambda t: t.float().cpu().numpy().astype(np.float64)
    at, ml = layer.self_attn, layer.mlp
    wq, wk, wv, wo = f64(at.q_proj), f64(at.k_proj), f64(at.v_proj), f64(at.o_proj)
    wg, wu, wd = f64(ml.gate_proj), f64(ml.up_proj), f64(ml.down_proj)

    def norm(s):
        return rb(s / np.sqrt((s * s).mean(axis=1, keepdims=True) + cfg.rms_norm_eps))

    for b in range(B):
        h0 = x[b].astype(np.float64)
        n1 = norm(h0)
        q, k, v = rb(n1 @ wq.T), rb(n1 @ wk.T), rb(n1 @ wv.T)
        attn = rb(R.attention_per_head(q, k, v, num_heads=8, num_kv_heads=2, head_dim=64, causal=True, dtype=np.float64,
                                       round_rope_bf16=True))
        h1 = rb(h0 + rb(attn @ wo.T))
        n2 = norm(h1)
        g, u = n2 @ wg.T, n2 @ wu.T
        m = rb(rb(g / (1.0 + np.exp(-g)) * u) @ wd.T)
        ref = rb(h1 + m)
        err = np.abs(got[b] - ref).max()
        # the attention path's 2e-2 plus two bf16 ulps at the largest magnitude: a value that sits near a rounding
        # boundary may round the other way in the kernel and its neighbours downstream
        assert err <= 2e-2 + np.abs(ref).max() * 2.0 ** -7, (err, np.abs(ref).max())

    layer2 = LLaMADecoderLayerBF16(cfg)
    plain = layer2(layer(tx))
    res, pend = layer.forward_parts(tx)
    res2, pend2 = layer2.forward_parts(res, pending=pend)
    assert torch.equal(res2 + pend2, plain)


def test_graphed_decoder_layer_equals_eager(lib):
    """The block captured into a CUDA graph returns the bits of the eager block, call after call."""
    from baranet_bdml_b200.layers import GraphedDecoderLayerBF16, LLaMAConfig, LLaMADecoderLayerBF16
    cfg = LLaMAConfig(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, intermediate_size=1408,
                      num_hidden_layers=1)
    np.random.seed(21)
    layer = LLaMADecoderLayerBF16(cfg)
    g = torch.Generator(device="cuda").manual_seed(1)
    xs = [torch.randn((2, 160, 512), generator=g, device="cuda").to(torch.bfloat16) for _ in range(3)]
    graphed = GraphedDecoderLayerBF16(layer, xs[0])
    for x in xs:
        res_e, mlp_e = layer.forward_parts(x)
        res_g, mlp_g = graphed(x)
        torch.cuda.synchronize()
        assert torch.equal(res_e, res_g) and torch.equal(mlp_e, mlp_g)


@pytest.mark.parametrize("M,N,K", [(1, 8, 8), (64, 2048, 2048), (64, 256, 2048), (17, 2048, 5632), (128, 1000, 520),
                                   (64, 32000, 2048), (130, 136, 264)])
def test_small_m_gemm(lib, M, N, K):
    """The split-K form for few rows: against fp64 on the same operands, equal run to run (fixed summation order), and
    within one bf16 ulp of the large-tile kernel."""
    from baranet_bdml_b200 import ops
    rng = np.random.default_rng(M * 3 + N + K)
    a = R.round_bf16(rng.standard_normal((M, K), dtype=np.float32))
    bt = R.round_bf16((rng.standard_normal((N, K)) * 0.05).astype(np.float32))
    ta, tb = torch.from_numpy(a).cuda().to(torch.bfloat16), torch.from_numpy(bt).cuda().to(torch.bfloat16)
    got = ops.gemm_bf16_nt_small_m(ta, tb)
    again = ops.gemm_bf16_nt_small_m(ta, tb)
    big = ops.gemm_bf16_nt(ta, tb)
    torch.cuda.synchronize()
    assert torch.equal(got, again)
    ref = a.astype(np.float64) @ bt.astype(np.float64).T
    scale = max(np.abs(ref).max(), 1e-30)
    assert np.abs(got.float().cpu().numpy() - ref).max() <= scale * 2.0 ** -8
    assert float((got.float() - big.float()).abs().max()) <= scale * 2.0 ** -7


@pytest.mark.parametrize("B,S,off", [(2, 200, 0), (1, 128, 0), (3, 77, 5)])
def test_fused_qkv_projection_with_rope_and_cache_append(lib, B, S, off):
    """bn_gemm_qkv_rope_bf16 against the separate launches it replaces: q and v are the bits of the plain GEMM; the
    rotated K (rotated from the fp32 accumulators, one rounding) is within one bf16 ulp of the fp64 rotation of the
    fp64 product; the cache pages hold that same K and V at positions off .. off + S - 1; the per-tile norm maxima
    bound the stored keys; and the attention that follows matches the unfused path within the bf16 gate."""
    from baranet_bdml_b200 import ops
    from baranet_bdml_b200.kv_cache import PagedKVCache, PAGE_TOKENS
    Hq, Hkv, D, hidden = 8, 2, 64, 256
    rng = np.random.default_rng(S + off)
    x = R.round_bf16(rng.standard_normal((B * S, hidden), dtype=np.float32))
    wq = R.round_bf16((rng.standard_normal((Hq * D, hidden)) * 0.06).astype(np.float32))
    wk = R.round_bf16((rng.standard_normal((Hkv * D, hidden)) * 0.06).astype(np.float32))
    wv = R.round_bf16((rng.standard_normal((Hkv * D, hidden)) * 0.06).astype(np.float32))
    tx = torch.from_numpy(x).cuda().to(torch.bfloat16)
    tq, tk, tv = (torch.from_numpy(w).cuda().to(torch.bfloat16) for w in (wq, wk, wv))
    wqkv = torch.cat([tq, tk, tv], 0).contiguous()
    max_pages = (S + off + PAGE_TOKENS - 1) // PAGE_TOKENS
    cache = PagedKVCache(B * max_pages + 3, B, max_pages, Hkv, D)
    perm = rng.permutation(B * max_pages + 3)[: B * max_pages].astype(np.int32).reshape(B, max_pages)
    cache.page_table.copy_(torch.from_numpy(perm))
    ws = ops.prefill_workspace(B, S, Hq, Hkv, D)
    ops.prefill_table(ws, B, S, Hkv, D, 10000.0, off)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    q, v = ops.gemm_qkv_rope_bf16(tx, wqkv, B, S, Hq, Hkv, D, ws, position_offset=off, cache=cache, error_word=err)
    out = ops.attn_prefill_bf16(q, None, v, position_offset=off, workspace=ws, reuse_rotated_k=True)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ws.status()
    # q, v: the plain GEMM's bits
    assert torch.equal(q.view(B * S, -1), ops.gemm_bf16_nt(tx, tq))
    assert torch.equal(v.view(B * S, -1), ops.gemm_bf16_nt(tx, tv))
    # rotated K in the cache pages against fp64
    k64 = x.astype(np.float64) @ wk.astype(np.float64).T                       # (B*S, Hkv*D)
    pool = cache.pool.float().cpu().numpy()
    vq = v.float().cpu().numpy().reshape(B, S, Hkv, D)
    worst = 0.0
    for b in range(B):
        pos = np.arange(S) + off
        i = np.arange(D // 2)
        freq = (1.0 / np.power(np.float32(10000.0), (2 * i).astype(np.float32) / np.float32(D))).astype(np.float32)
        ang = (pos[:, None].astype(np.float32) * freq[None]).astype(np.float64)
        kb = k64[b * S:(b + 1) * S].reshape(S, Hkv, D // 2, 2)
        rot = np.empty_like(kb)
        rot[..., 0] = kb[..., 0] * np.cos(ang)[:, None] - kb[..., 1] * np.sin(ang)[:, None]
        rot[..., 1] = kb[..., 0] * np.sin(ang)[:, None] + kb[..., 1] * np.cos(ang)[:, None]
        rot = rot.reshape(S, Hkv, D)
        pages, slots = perm[b][pos // PAGE_TOKENS], pos % PAGE_TOKENS
        got_k = pool[pages, :, 0, slots, :]                                    # (S, Hkv, D)
        got_v = pool[pages, :, 1, slots, :]
        worst = max(worst, np.abs(got_k - rot).max() / max(np.abs(rot).max(), 1e-30))
        assert np.array_equal(got_v, vq[b])
    assert worst <= 2.0 ** -8
    # the attention that follows, against the unfused path (separate GEMMs, K rotated from its bf16 rounding)
    k_plain = ops.gemm_bf16_nt(tx, tk).view(B, S, Hkv, D)
    ref = ops.attn_prefill_bf16(q, k_plain, v, position_offset=off)
    torch.cuda.synchronize()
    assert float((out.float() - ref.float()).abs().max()) <= 2e-2


@pytest.mark.parametrize("M,N,K", [(1, 8, 256), (16, 2048, 2048), (2, 2560, 2048), (16, 2048, 5632), (5, 32000, 2048),
                                   (13, 264, 512)])
def test_skinny_gemm(lib, M, N, K):
    """The weight-streaming product for at most 16 rows against fp64 on the same operands (one bf16 ulp at the largest
    magnitude), equal run to run, and split into three column ranges equal to the unsplit result."""
    from baranet_bdml_b200 import ops
    rng = np.random.default_rng(M + N + K)
    a = R.round_bf16(rng.standard_normal((M, K), dtype=np.float32))
    bt = R.round_bf16((rng.standard_normal((N, K)) * 0.05).astype(np.float32))
    ta, tb = torch.from_numpy(a).cuda().to(torch.bfloat16), torch.from_numpy(bt).cuda().to(torch.bfloat16)
    got = ops.gemm_bf16_nt_skinny(ta, tb)
    again = ops.gemm_bf16_nt_skinny(ta, tb)
    torch.cuda.synchronize()
    assert torch.equal(got, again)
    ref = a.astype(np.float64) @ bt.astype(np.float64).T
    assert np.abs(got.float().cpu().numpy() - ref).max() <= max(np.abs(ref).max(), 1e-30) * 2.0 ** -8
    if N >= 24:
        n0 = (N // 3) // 8 * 8
        n1 = 8
        parts = ops.gemm_bf16_nt_skinny(ta, tb, (n0, n1, N - n0 - n1))
        torch.cuda.synchronize()
        assert torch.equal(torch.cat(parts, dim=1), got)


def test_skinny_swiglu(lib):
    from baranet_bdml_b200 import ops
    rng = np.random.default_rng(77)
    M, K, inter = 16, 2048, 5632
    x = R.round_bf16(rng.standard_normal((M, K), dtype=np.float32))
    wg = R.round_bf16((rng.standard_normal((inter, K)) * 0.03).astype(np.float32))
    wu = R.round_bf16((rng.standard_normal((inter, K)) * 0.03).astype(np.float32))
    tx, tg, tu = (torch.from_numpy(t).cuda().to(torch.bfloat16) for t in (x, wg, wu))
    got = ops.gemm_swiglu_bf16_nt_skinny(tx, tg, tu).float().cpu().numpy()
    g = x.astype(np.float64) @ wg.astype(np.float64).T
    u = x.astype(np.float64) @ wu.astype(np.float64).T
    ref = g / (1.0 + np.exp(-g)) * u
    assert np.abs(got - ref).max() <= max(np.abs(ref).max(), 1e-30) * 2.0 ** -8
    assert lib.bn_gemm_bf16_nt_skinny(tx.data_ptr(), tg.data_ptr(), 17, inter, K, tx.data_ptr(), inter, None, 0, None, None) != 0


@pytest.mark.parametrize("M,Hq,Hkv,D,hidden", [(16, 32, 4, 64, 2048), (3, 4, 2, 64, 256), (7, 6, 3, 32, 512)])
def test_skinny_qkv_with_cache_append(lib, M, Hq, Hkv, D, hidden):
    """One launch for the q, k and v projections of a decode step with RoPE(K) and the cache append against the
    two-launch path (three-output skinny GEMM, then bn_kv_append): q equal, and every page of the cache equal bit for
    bit - including rows whose position is out of the page table's range, which both paths skip."""
    from baranet_bdml_b200 import ops
    from baranet_bdml_b200.kv_cache import PagedKVCache
    rng = np.random.default_rng(M * 1000 + hidden)
    x = torch.from_numpy(R.round_bf16(rng.standard_normal((M, hidden), dtype=np.float32))).cuda().to(torch.bfloat16)
    w = torch.from_numpy(R.round_bf16((rng.standard_normal(((Hq + 2 * Hkv) * D, hidden)) * 0.05).astype(np.float32)))
    w = w.cuda().to(torch.bfloat16)
    pages_per = 6                                                      # 96 positions per sequence
    pos = rng.integers(0, pages_per * 16, (M,)).astype(np.int32)
    if M > 4:
        pos[1] = pages_per * 16 + 5                                    # past the last page: skipped
        pos[2] = -1
    seq = rng.permutation(M).astype(np.int32)
    caches = []
    for _ in range(2):
        c = PagedKVCache(M * pages_per + 2, M, pages_per, Hkv, D)
        c.page_table.copy_(torch.from_numpy(rng.permutation(M * pages_per + 2)[: M * pages_per].astype(np.int32)
                                            .reshape(M, pages_per)))
        c.pool.zero_()
        caches.append(c)
    caches[1].page_table.copy_(caches[0].page_table)
    seq_t, pos_t = torch.from_numpy(seq).cuda(), torch.from_numpy(pos).cuda()
    q1, k1, v1 = ops.gemm_bf16_nt_skinny(x, w, (Hq * D, Hkv * D, Hkv * D))
    caches[0].append(seq_t, pos_t, k1, v1)
    q2 = ops.gemm_qkv_append_bf16_skinny(x, w, caches[1], seq_t, pos_t, Hq)
    torch.cuda.synchronize()
    assert torch.equal(q1, q2)
    assert torch.equal(caches[0].pool, caches[1].pool)
    assert float(caches[1].pool.float().abs().max()) > 0

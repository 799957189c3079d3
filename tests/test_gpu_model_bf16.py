"""The bf16 model with a paged KV cache: one-token decode steps against whole-sequence recomputation (what the
reference's generate() does, mygrad/llama/llama_model.py:136-144), on the same weights."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def tiny_model(seed=0):
    from baranet_bdml_b200.layers import LLaMAConfig
    from baranet_bdml_b200.model import LLaMAModelBF16
    cfg = LLaMAConfig(vocab_size=1000, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256)
    np.random.seed(seed)
    return LLaMAModelBF16(cfg)


def test_cached_decode_matches_recomputation(lib):
    """Logits of every new position from prefill + decode steps (K/V from the cache, one query row) against the last
    row of a whole-sequence forward over the same tokens.  Both run bf16 kernels with different reduction orders, so
    the gate is a tolerance: 3e-2 of the logit range."""
    model = tiny_model()
    rng = np.random.default_rng(1)
    B, S, new = 3, 37, 6
    ids = torch.from_numpy(rng.integers(3, 1000, (B, S + new)).astype(np.int32)).cuda()
    logits = model.prefill(ids[:, :S].contiguous(), S + new)
    for t in range(new + 1):
        full = model(ids[:, :S + t].contiguous())[:, -1]             # recompute everything, keep the last row
        torch.cuda.synchronize()
        scale = float(full.abs().max())
        assert float((logits - full).abs().max()) <= 3e-2 * scale, (t, float((logits - full).abs().max()), scale)
        if t < new:
            logits = model.decode_step(ids[:, S + t].contiguous())
    assert int(model.caches[0].seq_lens[0]) == S + new


def test_generate_greedy_equals_recompute_generate(lib):
    """Greedy generate() with the cache picks the tokens that recomputing the whole sequence would pick, as long as
    the best two logits of the recomputed row are further apart than the bf16 tolerance of the two paths."""
    model = tiny_model(3)
    rng = np.random.default_rng(4)
    prompt = rng.integers(3, 1000, (2, 20)).astype(np.int32)
    out = model.generate(prompt, max_new_tokens=5)
    assert all(len(o) >= 20 for o in out)
    for b in range(2):
        seq = list(prompt[b])
        for tok in out[b][20:]:
            full = model(torch.tensor([seq], dtype=torch.int32, device="cuda"))[0, -1]
            top2 = torch.topk(full, 2).values
            if float(top2[0] - top2[1]) > 3e-2 * float(full.abs().max()):
                assert int(torch.argmax(full)) == tok
            seq.append(tok)


def test_graphed_decode_step_equals_eager(lib):
    """The decode step replayed from a CUDA graph gives the bits of the eager step, position after position."""
    rng = np.random.default_rng(6)
    ids = torch.from_numpy(rng.integers(3, 1000, (2, 30)).astype(np.int32)).cuda()
    toks = torch.from_numpy(rng.integers(3, 1000, (4, 2)).astype(np.int32)).cuda()
    eager = tiny_model(5)
    eager.prefill(ids, 64)
    want = [eager.decode_step(t).clone() for t in toks]
    graphed = tiny_model(5)                       # same seed: same weights
    graphed.prefill(ids, 64)
    step = graphed.capture_decode_step()
    for t, w in zip(toks, want):
        logits, nxt = step(t)
        torch.cuda.synchronize()
        assert torch.equal(logits, w)
        assert torch.equal(nxt, graphed.argmax(w))
    assert int(graphed.caches[0].seq_lens[0]) == 34


def test_model_rejects_bad_ids(lib):
    model = tiny_model()
    with pytest.raises(IndexError):
        model.embed(torch.tensor([5, 1000], dtype=torch.int32, device="cuda"))


def test_model_logits_against_staged_fp64(lib):
    """The model's whole-sequence forward (teacher-forced logits of a 2-layer reduced TinyLLaMA: embedding gather,
    two blocks with the deferred residual add, final norm, lm_head) against an fp64 restatement assembled from the
    oracle's pieces, with a bf16 rounding wherever a kernel rounds - the model's own plumbing (casts, the pending
    residual, the last-position slice of prefill) checked against something that is not the model."""
    from oracle import ref_attention as R
    model = tiny_model(7)
    cfg = model.config
    rng = np.random.default_rng(8)
    B, S = 2, 70
    ids_np = rng.integers(0, cfg.vocab_size, (B, S)).astype(np.int32)
    ids = torch.from_numpy(ids_np).cuda()
    got = model(ids).float().cpu().numpy()                              # (B, S, vocab)
    got_last = model.prefill(ids, S + 4).float().cpu().numpy()          # prompt pass: last position only

    rb = lambda a: R.round_bf16(np.asarray(a, dtype=np.float32)).astype(np.float64)
    f64 = lambda t: t.float().cpu().numpy().astype(np.float64)
    table = f64(model.embed_tokens)
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim

    def norm(s, w):
        return rb(s / np.sqrt((s * s).mean(axis=1, keepdims=True) + cfg.rms_norm_eps) * w)

    for b in range(B):
        h = rb(table[ids_np[b]])                                        # gather (fp32 rows), cast to bf16
        pending = None
        for layer in model.layers:
            at, ml = layer.self_attn, layer.mlp
            s0 = h if pending is None else rb(h + pending)              # the fused add of the previous block's MLP output
            n1 = norm(s0, f64(layer.input_layernorm_weight))
            q, k, v = rb(n1 @ f64(at.q_proj).T), rb(n1 @ f64(at.k_proj).T), rb(n1 @ f64(at.v_proj).T)
            attn = rb(R.attention_per_head(q, k, v, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, causal=True,
                                           dtype=np.float64, round_rope_bf16=True))
            s1 = rb(s0 + rb(attn @ f64(at.o_proj).T))
            n2 = norm(s1, f64(layer.post_attention_layernorm_weight))
            g, u = n2 @ f64(ml.gate_proj).T, n2 @ f64(ml.up_proj).T
            pending = rb(rb(g / (1.0 + np.exp(-g)) * u) @ f64(ml.down_proj).T)
            h = s1
        final = norm(rb(h + pending), f64(model.norm_weight))
        ref = rb(final @ f64(model.lm_head).T)                          # logits leave the GEMM as bf16
        scale = np.abs(ref).max()
        err = np.abs(got[b] - ref).max()
        # two blocks of the decoder-layer gate (2e-2 + two bf16 ulps each) carried through a norm and one more GEMM
        assert err <= 3e-2 * scale, (b, err, scale)
        assert np.abs(got_last[b] - ref[-1]).max() <= 3e-2 * scale


def test_model_status_reads_the_gemm_error_word(lib):
    """Every projection GEMM of the model reports into one error word per device; `status()` is quiet after an ordinary
    generation, raises once when the word is set (here by hand: nothing is made to hang) and clears it."""
    from baranet_bdml_b200 import ops
    model = tiny_model(9)
    ids = torch.from_numpy(np.random.default_rng(2).integers(3, 1000, (2, 40)).astype(np.int32)).cuda()
    model.prefill(ids, 48)
    model.decode_step(ids[:, 0].contiguous())
    model.status()
    word = ops._gemm_err[torch.cuda.current_device()]
    word.fill_(-6)
    with pytest.raises(RuntimeError):
        model.status()
    model.status()
    assert int(word.item()) == 0

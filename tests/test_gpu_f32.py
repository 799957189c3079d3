"""fp32 path vs the oracle, through the C ABI (TensorF / AGTensor mirror the
reference's bten / mygrad surface, so these read like the reference's own
test_llama.py — with assertions).  Gate (fp32 path): max|d| / max|ref| <= 1e-5."""
import numpy as np
import pytest
import torch

from oracle import ref_attention as R

pytestmark = pytest.mark.gpu

GATE = 1e-5


def nerr(a, b):
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / max(np.abs(b).max(), 1e-30))


@pytest.fixture(scope="module")
def T(lib):
    from baranet_bdml_b200 import tensor
    return tensor


@pytest.fixture(scope="module")
def dev_inv_freq(T):
    """The device's own frequency table (CUDA powf), read back through bn_rope_f32:
    rotating (1, 0) pairs at position 1 yields (cos f_i, sin f_i)."""
    out = {}
    for D in (32, 64):
        x = np.zeros((1, D), dtype=np.float32)
        x[0, 0::2] = 1.0
        t = T.TensorF(1, D)
        t.copy_from_numpy(x)
        y = t.rope(1, D, 10000.0).to_numpy()
        out[D] = np.arctan2(y[0, 1::2].astype(np.float64), y[0, 0::2].astype(np.float64))
    return out


def test_inv_freq_matches_cpu_table(dev_inv_freq, cref):
    for D in (32, 64):
        cpu = cref.inv_freq(D).astype(np.float64)
        assert np.abs(dev_inv_freq[D] - cpu).max() / cpu.max() < 1e-6


@pytest.mark.parametrize("M,K,N", [(128, 2048, 256), (4, 128, 64), (33, 70, 65), (1, 64, 1), (130, 16, 200)])
def test_mm_matches_reference_order(T, cref, M, K, N):
    rng = np.random.default_rng(1)
    a = rng.standard_normal((M, K), dtype=np.float32)
    b = rng.standard_normal((K, N), dtype=np.float32)
    ta, tb = T.TensorF(M, K), T.TensorF(K, N)
    ta.copy_from_numpy(a)
    tb.copy_from_numpy(b)
    got = (ta @ tb).to_numpy()
    import ctypes as C
    ref = np.empty((M, N), dtype=np.float32)
    fp = C.POINTER(C.c_float)
    cref.cpu().ref_mm_f32(a.ctypes.data_as(fp), C.c_long(K), C.c_long(1), b.ctypes.data_as(fp), C.c_long(N),
                          C.c_long(1), ref.ctypes.data_as(fp), C.c_int(M), C.c_int(K), C.c_int(N))
    assert np.array_equal(got, ref), nerr(got, ref)   # same FMA chain -> same bits


def test_mm_transposed_and_sliced_views(T):
    rng = np.random.default_rng(2)
    a = rng.standard_normal((40, 96), dtype=np.float32)
    b = rng.standard_normal((50, 96), dtype=np.float32)
    ta, tb = T.TensorF(40, 96), T.TensorF(50, 96)
    ta.copy_from_numpy(a)
    tb.copy_from_numpy(b)
    got = (ta[4:36, 32:96] @ tb.T[32:96, 1:50]).to_numpy()
    ref = a[4:36, 32:96].astype(np.float64) @ b.T[32:96, 1:50].astype(np.float64)
    assert nerr(got, ref) < 1e-6


@pytest.mark.parametrize("rows,cols,D,off", [(4, 64, 32, 0), (128, 2048, 64, 0), (128, 256, 64, 7), (3, 128, 64, 2040)])
def test_rope(T, cref, rows, cols, D, off):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((rows, cols), dtype=np.float32)
    t = T.TensorF(rows, cols)
    t.copy_from_numpy(x)
    got = t.rope(off, D, 10000.0).to_numpy()
    ref = cref.rope(x, D, 10000.0, off)
    # angles are fp32 products position*freq; a last-bit difference between CUDA's and glibc's
    # powf moves the angle by position * 2^-24 relative
    tol = 1e-6 + (rows + off) * 2.0 ** -23
    assert nerr(got, ref) < tol


CASES = [  # S, Hq, Hkv, D, offset, causal
    (128, 32, 4, 64, 0, True),     # the layer shape of BASELINE config 1
    (4, 4, 2, 32, 0, True),        # the reference's own test shape (test_llama.py:142-165)
    (2, 4, 2, 32, 0, True),
    (1, 32, 4, 64, 0, True),
    (17, 8, 2, 64, 3, True),
    (65, 8, 8, 32, 0, False),
    (130, 4, 1, 64, 0, True),
]


@pytest.mark.parametrize("S,Hq,Hkv,D,off,causal", CASES)
@pytest.mark.parametrize("mode", ["collapsed", "per_head"])
def test_attention_core_f32(T, cref, dev_inv_freq, S, Hq, Hkv, D, off, causal, mode):
    from baranet_bdml_b200 import _lib
    rng = np.random.default_rng(S * 131 + Hq)
    q = rng.standard_normal((S, Hq * D), dtype=np.float32)
    k = rng.standard_normal((S, Hkv * D), dtype=np.float32)
    v = rng.standard_normal((S, Hkv * D), dtype=np.float32)
    tq, tk, tv = T.TensorF(S, Hq * D), T.TensorF(S, Hkv * D), T.TensorF(S, Hkv * D)
    for t, a in ((tq, q), (tk, k), (tv, v)):
        t.copy_from_numpy(a)
    scale = 1.0 / np.sqrt(D)
    hm = _lib.BN_HEADS_COLLAPSED if mode == "collapsed" else _lib.BN_HEADS_PER_HEAD
    got = tq.attention_fused(tk, tv, scale, causal, off, num_heads=Hq, num_kv_heads=Hkv, head_dim=D,
                             heads_mode=hm).to_numpy()
    inv = dev_inv_freq[D].astype(np.float32)
    if mode == "collapsed":
        ref = cref.attention_collapsed(q, k, v, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, position_offset=off,
                                       causal=causal, inv_freq=inv)
        ref64 = R.attention_collapsed(q, k, v, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, position_offset=off,
                                      causal=causal, dtype=np.float64, inv_freq=inv)
    else:
        ref64 = R.attention_per_head(q, k, v, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, position_offset=off,
                                     causal=causal, dtype=np.float64, inv_freq=inv)
        ref = ref64.astype(np.float32)
    assert nerr(got, ref) < GATE, (nerr(got, ref), nerr(got, ref64))
    assert nerr(got, ref64) < 2e-5


def test_layer_config1_matches_oracle(T, cref, dev_inv_freq):
    """BASELINE config 1: one TinyLLaMA attention layer, fp32, S=128, through the
    mirrored GroupedQueryAttention API with injected seeded weights."""
    from baranet_bdml_b200.layers import GroupedQueryAttention, LLaMAConfig
    from baranet_bdml_b200.tensor import AGTensor
    cfg = LLaMAConfig()
    rng = np.random.default_rng(0)
    S, hid, Hq, Hkv, D = 128, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    x = rng.standard_normal((S, hid), dtype=np.float32)
    wq = (rng.standard_normal((hid, Hq * D)) * 0.02).astype(np.float32)
    wk = (rng.standard_normal((hid, Hkv * D)) * 0.02).astype(np.float32)
    wv = (rng.standard_normal((hid, Hkv * D)) * 0.02).astype(np.float32)
    wo = (rng.standard_normal((Hq * D, hid)) * 0.02).astype(np.float32)
    attn = GroupedQueryAttention(cfg, is_cuda=True)
    attn.q_proj, attn.k_proj, attn.v_proj, attn.o_proj = (AGTensor(w, is_cuda=True) for w in (wq, wk, wv, wo))
    out = attn(AGTensor(x, is_cuda=True)).numpy()
    assert out.shape == (S, hid)
    inv = dev_inv_freq[D].astype(np.float32)
    ref = cref.gqa_layer(x, wq, wk, wv, wo, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, inv_freq=inv)
    assert nerr(out, ref) < GATE, nerr(out, ref)
    ref64 = R.gqa_layer_collapsed(x, wq, wk, wv, wo, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, dtype=np.float64,
                                  inv_freq=inv)
    assert nerr(out, ref64) < 2e-5


def test_layer_matches_reference_cuda_ops(T, cref):
    """Same inputs through the reference's OWN CUDA operators (compiled from the
    reference tree into oracle/_ref) and through the fused layer."""
    if not cref.gpu_available():
        pytest.skip("oracle/_ref not built (needs the reference tree at build time)")
    from baranet_bdml_b200.layers import GroupedQueryAttention, LLaMAConfig
    from baranet_bdml_b200.tensor import AGTensor
    for cfg, S in ((LLaMAConfig(), 128), (LLaMAConfig(vocab_size=1000, hidden_size=128, intermediate_size=256,
                                                     num_hidden_layers=2, num_attention_heads=4,
                                                     num_key_value_heads=2), 4)):
        rng = np.random.default_rng(5)
        hid, Hq, Hkv, D = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        x = rng.standard_normal((S, hid), dtype=np.float32)
        ws = [(rng.standard_normal(s) * 0.02).astype(np.float32)
              for s in ((hid, Hq * D), (hid, Hkv * D), (hid, Hkv * D), (Hq * D, hid))]
        attn = GroupedQueryAttention(cfg, is_cuda=True)
        attn.q_proj, attn.k_proj, attn.v_proj, attn.o_proj = (AGTensor(w, is_cuda=True) for w in ws)
        out = attn(AGTensor(x, is_cuda=True)).numpy()
        ref = cref.gpu_gqa_layer(x, *ws, num_heads=Hq, num_kv_heads=Hkv, head_dim=D)
        assert nerr(out, ref) < GATE, nerr(out, ref)


def test_host_tensor_ops_raise(T):
    a = T.TensorF(4, 4, is_cuda=False)
    with pytest.raises(RuntimeError, match="only GPU implementation available"):
        a @ a
    with pytest.raises(RuntimeError, match="only GPU implementation available"):
        a.rope()

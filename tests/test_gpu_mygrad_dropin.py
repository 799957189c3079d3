"""The reference's OWN attention layer, unmodified, on the new kernels.

`oracle/_ref/` (built by `make -C oracle bten REF=<reference tree>`) holds the superset `bten` module - the
reference's pybind11 shim and operators compiled where they lie, plus the entries of
baranet_bdml_b200/binding/bten_b200.cu - and the reference's `mygrad` package staged unmodified.  The test
imports that `mygrad`, runs `GroupedQueryAttention` (mygrad/llama/llama_layers.py:140-188) once as the reference
wrote it and once with `__call__` rebound to the fused entry (baranet_bdml_b200/mygrad_dropin.py), in the same
process on the same weights, and compares: max|diff| / max|ref| <= 1e-5.  Shapes: BASELINE config 1 and the
reference's own test shapes (test_llama.py:142-199: hidden 128, 4 query / 2 KV heads -> head_dim 32, 2 to 4 rows).
Skipped where oracle/_ref has not been built."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BTEN_DIR = os.path.join(ROOT, "oracle", "_ref", "bten_b200")
PYREF = os.path.join(ROOT, "oracle", "_ref", "pyref")
GATE = 1e-5


@pytest.fixture(scope="module")
def ref(lib):
    if not (os.path.isdir(BTEN_DIR) and os.path.isdir(os.path.join(PYREF, "mygrad"))):
        pytest.skip("oracle/_ref/bten_b200 and oracle/_ref/pyref are not built (make -C oracle bten REF=...)")
    for d in (PYREF, BTEN_DIR):
        if d not in sys.path:
            sys.path.insert(0, d)
    import bten
    assert bten.has_b200_attention
    from mygrad.engine import AGTensor
    import mygrad.llama.llama_layers as layers
    from mygrad.llama.llama_config import LLaMAConfig
    return bten, AGTensor, layers, LLaMAConfig


def _layer(ref, hidden, heads, kv_heads, seed, std):
    bten, AGTensor, layers, LLaMAConfig = ref
    cfg = LLaMAConfig()
    cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads = hidden, heads, kv_heads
    attn = layers.GroupedQueryAttention(cfg, is_cuda=True)
    rng = np.random.default_rng(seed)
    kv = kv_heads * cfg.head_dim
    # weights are plain attributes of the layer (llama_layers.py:66-69)
    attn.q_proj = AGTensor((rng.standard_normal((hidden, hidden)) * std).astype(np.float32), is_cuda=True)
    attn.k_proj = AGTensor((rng.standard_normal((hidden, kv)) * std).astype(np.float32), is_cuda=True)
    attn.v_proj = AGTensor((rng.standard_normal((hidden, kv)) * std).astype(np.float32), is_cuda=True)
    attn.o_proj = AGTensor((rng.standard_normal((hidden, hidden)) * std).astype(np.float32), is_cuda=True)
    return attn, rng


def _both(ref, attn, x_np, **kw):
    from baranet_bdml_b200 import mygrad_dropin
    bten, AGTensor, layers, _ = ref
    x = AGTensor(x_np, is_cuda=True)
    want = attn(x, **kw).numpy()
    mygrad_dropin.install(layers)
    try:
        assert layers.GroupedQueryAttention.__call__ is mygrad_dropin.fused_call
        got_t = attn(x, **kw)
        got = got_t.numpy()
    finally:
        mygrad_dropin.uninstall(layers)
    assert type(got_t).__name__ == "AGTensor" and isinstance(got_t.data, bten.TensorF)
    assert got.shape == want.shape and got.dtype == want.dtype
    return got, want


def test_config1_layer_through_the_reference_api(ref):
    attn, rng = _layer(ref, 2048, 32, 4, seed=1, std=0.02)
    x = rng.standard_normal((128, 2048)).astype(np.float32)
    got, want = _both(ref, attn, x)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() / np.abs(want).max() <= GATE


@pytest.mark.parametrize("rows", [2, 3, 4, 33])
@pytest.mark.parametrize("offset,causal", [(0, True), (5, True), (0, False)])
def test_reference_test_shapes(ref, rows, offset, causal):
    attn, rng = _layer(ref, 128, 4, 2, seed=rows * 10 + offset, std=0.2)
    x = rng.standard_normal((rows, 128)).astype(np.float32)
    got, want = _both(ref, attn, x, position_offset=offset, use_causal_mask=causal)
    assert np.abs(got - want).max() / np.abs(want).max() <= GATE


def test_decoder_layer_and_model_pick_up_the_rebound_layer(ref):
    """LLaMADecoderLayer (llama_layers.py:238-296) is untouched: it finds the fused attention through the class."""
    from baranet_bdml_b200 import mygrad_dropin
    bten, AGTensor, layers, LLaMAConfig = ref
    cfg = LLaMAConfig()
    cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size = 128, 4, 2, 256
    block = layers.LLaMADecoderLayer(cfg, is_cuda=True)
    x = AGTensor(np.random.default_rng(3).standard_normal((4, 128)).astype(np.float32), is_cuda=True)
    want = block(x, position_offset=0).numpy()
    mygrad_dropin.install(layers)
    try:
        got = block(x, position_offset=0).numpy()
    finally:
        mygrad_dropin.uninstall(layers)
    assert np.abs(got - want).max() / np.abs(want).max() <= GATE


def test_replacement_operators_against_the_reference_operators(ref):
    bten, AGTensor, layers, _ = ref
    rng = np.random.default_rng(7)

    def tensor(a):
        t = bten.TensorF(a.shape[0], a.shape[1], True)
        t.copy_from_numpy(a)
        return t

    a, b = rng.standard_normal((70, 96)).astype(np.float32), rng.standard_normal((96, 50)).astype(np.float32)
    ta, tb = tensor(a), tensor(b)
    assert np.array_equal(ta.matmul_b200(tb).to_numpy(), (ta @ tb).to_numpy())                 # same k-ascending chains
    x = tensor(rng.standard_normal((9, 256)).astype(np.float32))
    assert np.array_equal(x.rope_b200(3, 64, 10000.0).to_numpy(), x.rope(3, 64, 10000.0).to_numpy())
    w = tensor((1 + 0.1 * rng.standard_normal((1, 256))).astype(np.float32))
    assert np.array_equal(x.rmsnorm_b200(w, 1e-6).to_numpy(), x.rmsnorm(w, 1e-6).to_numpy())
    y = tensor(rng.standard_normal((9, 256)).astype(np.float32))
    total, normed = x.add_rmsnorm(y, w, 1e-6)
    assert np.array_equal(total.to_numpy(), (x + y).to_numpy())
    assert np.array_equal(normed.to_numpy(), (x + y).rmsnorm(w, 1e-6).to_numpy())
    logits = tensor(rng.standard_normal((6, 1000)).astype(np.float32))
    assert np.array_equal(logits.argmax_b200().to_numpy(), logits.argmax().to_numpy())
    table = rng.standard_normal((50, 64)).astype(np.float32)
    ids = np.array([[3, 0, 49, 7]], dtype=np.uint32)
    tids = bten.TensorU32(1, 4, True)
    tids.copy_from_numpy(ids)
    assert np.array_equal(tensor(table).gather_rows(tids).to_numpy(), table[ids[0]])


def test_errors_follow_the_reference_convention(ref):
    bten, AGTensor, layers, _ = ref
    host = bten.TensorF(4, 128, False)
    with pytest.raises(RuntimeError, match="only GPU implementation available"):
        host.attention_fused(host, host, 0.125, True, 0, num_heads=2, num_kv_heads=2, head_dim=64)
    dev = bten.TensorF(4, 128, True)
    with pytest.raises(RuntimeError, match="hidden size mismatch"):
        dev.attention_fused(dev, dev, 0.125, True, 0, num_heads=4, num_kv_heads=2, head_dim=64)


def test_the_reference_smoke_script_runs_unmodified_on_the_superset_module(ref):
    """test_llama.py of the reference (staged as it is) imports `bten` from ./build: here that is the superset."""
    script = os.path.join(PYREF, "test_llama.py")
    if not os.path.exists(script):
        pytest.skip("test_llama.py is not staged")
    res = subprocess.run([sys.executable, script], cwd=PYREF, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]

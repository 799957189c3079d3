"""The oracle against itself and against the committed golden vectors (CPU only).

The reference holds no golden vectors for this path; the fixtures under
tests/golden/ are outputs of the reference's own CUDA operators run on a B200
(see tests/golden/README.md)."""
import glob
import os

import numpy as np
import pytest

from oracle import ref_attention as R

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def nerr(a, b):
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / max(np.abs(b).max(), 1e-30))


def test_c_and_numpy_restatements_agree(cref):
    rng = np.random.default_rng(0)
    S, Hq, Hkv, D = 48, 8, 2, 32
    q = rng.standard_normal((S, Hq * D), dtype=np.float32)
    k = rng.standard_normal((S, Hkv * D), dtype=np.float32)
    v = rng.standard_normal((S, Hkv * D), dtype=np.float32)
    for off, causal in ((0, True), (3, True), (0, False)):
        a = cref.attention_collapsed(q, k, v, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, position_offset=off,
                                     causal=causal)
        b = R.attention_collapsed(q, k, v, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, position_offset=off,
                                  causal=causal, dtype=np.float64)
        assert nerr(a, b) < 1e-5
    assert np.array_equal(cref.inv_freq(64), R.rope_inv_freq(64))
    x = rng.standard_normal((9, 128), dtype=np.float32)
    assert nerr(cref.rope(x, 64, 10000.0, 5), R.rope(x, 5, 64)) < 1e-6
    assert nerr(cref.softmax(x, True, 2), R.softmax_rows(x, True, 2)) < 1e-6


def test_collapsed_equals_single_head_of_group_summed_queries():
    """The reference's layer (one softmax over all heads) == single-head attention with
    Q' = sum over the query heads of each KV group, head_dim = Hkv*D."""
    rng = np.random.default_rng(1)
    S, Hq, Hkv, D = 20, 8, 2, 16
    q = rng.standard_normal((S, Hq * D))
    k = rng.standard_normal((S, Hkv * D))
    v = rng.standard_normal((S, Hkv * D))
    a = R.attention_collapsed(q, k, v, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, dtype=np.float64)
    qr = R.rope(q, 0, D, dtype=np.float64).reshape(S, Hkv, Hq // Hkv, D).sum(2).reshape(S, Hkv * D)
    kr = R.rope(k, 0, D, dtype=np.float64)
    p = R.softmax_rows(qr @ kr.T / np.sqrt(D), True, 0, np.float64)
    o = (p @ v).reshape(S, Hkv, 1, D).repeat(Hq // Hkv, 2).reshape(S, Hq * D)
    assert np.abs(a - o).max() < 1e-12


def test_decode_is_last_row_of_prefill_in_the_oracle(cref):
    rng = np.random.default_rng(2)
    S, Hq, Hkv, D = 70, 8, 2, 64
    q = R.round_bf16(rng.standard_normal((S, Hq * D), dtype=np.float32))
    k = R.round_bf16(rng.standard_normal((S, Hkv * D), dtype=np.float32))
    v = R.round_bf16(rng.standard_normal((S, Hkv * D), dtype=np.float32))
    full, full_lse = R.attention_per_head(q, k, v, num_heads=Hq, num_kv_heads=Hkv, head_dim=D,
                                          round_rope_bf16=True, return_lse=True)
    n_pages = 8
    pt = rng.permutation(n_pages)[:5].astype(np.int32)[None]
    pool = R.kv_append(np.zeros((n_pages, Hkv, 2, 16, D), dtype=np.uint16), pt, np.arange(S), np.zeros(S, int), k, v,
                       head_dim=D)
    poolf = R.bf16_bits_to_f32(pool)
    for t in (0, 15, 16, 69):
        o, lse = R.decode_paged(q[t:t + 1], poolf, pt, np.array([t + 1]), num_heads=Hq, num_kv_heads=Hkv, head_dim=D,
                                return_lse=True)
        assert np.abs(o[0] - full[t]).max() < 1e-9
        assert np.abs(lse[0] - full_lse[t]).max() < 1e-9
    # plain-C decode agrees (it takes an already rotated query)
    qrot = R.round_bf16(R.rope(q[69:70], head_dim=D, positions=np.array([69])))
    oc, lc = cref.decode_paged(qrot, pool, pt, np.array([70], dtype=np.int32), num_heads=Hq, num_kv_heads=Hkv,
                               head_dim=D)
    assert np.abs(oc[0] - full[69]).max() < 1e-4


def test_sequence_split_plus_lse_combine_is_exact():
    rng = np.random.default_rng(3)
    L, Hq, Hkv, D, P = 96, 8, 2, 64, 3
    pool = R.round_bf16(rng.standard_normal((6, Hkv, 2, 16, D), dtype=np.float32))
    pt = np.arange(6, dtype=np.int32)[None]
    q = R.round_bf16(rng.standard_normal((1, Hq * D), dtype=np.float32))
    full, full_lse = R.decode_paged(q, pool, pt, np.array([L]), num_heads=Hq, num_kv_heads=Hkv, head_dim=D,
                                    return_lse=True)
    outs, lses = [], []
    for r in range(P + 1):     # the last shard is empty
        o, l = R.decode_paged(q, pool, pt, np.array([L]), num_heads=Hq, num_kv_heads=Hkv, head_dim=D,
                              return_lse=True, token_begin=np.array([r * 32]), token_end=np.array([(r + 1) * 32]))
        outs.append(o.reshape(Hq, D))
        lses.append(l.reshape(Hq))
    assert not np.isfinite(lses[-1]).any()
    o, l = R.lse_combine(np.stack(outs), np.stack(lses))
    assert np.abs(o.reshape(-1) - full[0]).max() < 1e-12
    assert np.abs(l - full_lse[0]).max() < 1e-12


def test_bf16_rounding_helpers():
    x = np.array([1.0, 1.00390625, 1.005859375, -2.5, 3.0e38, 0.0], dtype=np.float32)
    b = R.f32_to_bf16_bits(x)
    assert b[0] == 0x3F80
    assert b[1] == 0x3F80          # exactly half way: ties to even (down)
    assert b[2] == 0x3F81
    assert np.array_equal(R.bf16_bits_to_f32(R.f32_to_bf16_bits(R.round_bf16(x))), R.round_bf16(x))


def _golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "ref_cuda_*.npz")))


@pytest.mark.parametrize("path", _golden_files() or [None])
def test_oracle_matches_reference_cuda_golden(path, cref):
    """Pins the restatement: outputs of the reference's own CUDA operators on a B200."""
    if path is None:
        pytest.skip("no golden fixtures generated yet")
    g = np.load(path)
    kind = str(g["kind"])
    if kind == "argmax":
        assert np.array_equal(R.argmax_rows(g["x"]), g["out"]), path
        return
    if kind == "rmsnorm":
        # fp32 with the reference's own arithmetic order: bit for bit
        got = cref.rmsnorm(g["x"], g["w"], float(g["eps"]))
        assert np.array_equal(got, g["out"]), (path, nerr(got, g["out"]))
        return
    kw = dict(num_heads=int(g["Hq"]), num_kv_heads=int(g["Hkv"]), head_dim=int(g["D"]),
              position_offset=int(g["offset"]), causal=bool(g["causal"]), inv_freq=g["inv_freq"])
    if kind == "layer":
        got = cref.gqa_layer(g["x"], g["wq"], g["wk"], g["wv"], g["wo"], **kw)
    elif kind == "core":
        got = cref.attention_collapsed(g["q"], g["k"], g["v"], **kw)
    elif kind == "layer_seeded":
        import importlib.util
        spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
        mg = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mg)
        x, wq, wk, wv, wo = mg.layer_inputs_from_seed(int(g["seed"]), int(g["S"]), int(g["hidden"]), int(g["Hq"]),
                                                      int(g["Hkv"]), int(g["D"]))
        full = cref.gqa_layer(x, wq, wk, wv, wo, **kw)
        got = full[::int(g["sub_rows"]), ::int(g["sub_cols"])]
        err = float(np.abs(got.astype(np.float64) - g["out_sub"]).max() / float(g["out_absmax"]))
        assert err <= 1e-5, (path, err)
        return
    elif kind == "rope":
        got = cref.rope(g["x"], int(g["D"]), 10000.0, int(g["offset"]), inv_freq=g["inv_freq"])
    else:
        pytest.fail(kind)
    assert nerr(got, g["out"]) <= 1e-5, (path, nerr(got, g["out"]))


def test_rmsnorm_restatements_agree(cref):
    """The bit-faithful C restatement of op_rmsnorm against the exact-math numpy statement; residual form; hidden
    sizes that are not a multiple of the reference's 256 threads; one element; a zero row (eps alone)."""
    rng = np.random.default_rng(5)
    for rows, hidden in ((4, 2048), (3, 300), (2, 1), (1, 5000), (5, 256)):
        x = rng.standard_normal((rows, hidden), dtype=np.float32) * 3
        w = (1 + 0.2 * rng.standard_normal(hidden)).astype(np.float32)
        r = rng.standard_normal((rows, hidden), dtype=np.float32)
        want = R.rmsnorm(x, w, 1e-6)
        got = cref.rmsnorm(x, w, 1e-6)
        assert np.abs(got - want).max() <= 2e-6 * np.abs(want).max() + 1e-12
        s, y = cref.add_rmsnorm(x, r, w, 1e-6)
        assert np.array_equal(s, x + r)
        assert np.array_equal(y, cref.rmsnorm(x + r, w, 1e-6))      # the fused form IS add followed by norm
    z = np.zeros((2, 64), dtype=np.float32)
    assert np.array_equal(cref.rmsnorm(z, np.ones(64, np.float32), 1e-6), z)


def test_argmax_and_embed_restatements():
    """The sequential first-maximum rule against numpy's argmax (the same rule on NaN-free data) and its NaN / tie
    cases; the host gather."""
    rng = np.random.default_rng(9)
    x = rng.standard_normal((20, 300)).astype(np.float32)
    x[3, [5, 9]] = 50.0
    assert np.array_equal(R.argmax_rows(x)[:, 0], np.argmax(x, axis=1))
    y = np.array([[np.nan, 3.0, 1.0], [1.0, np.nan, 2.0], [-np.inf, -np.inf, -np.inf]], dtype=np.float32)
    assert list(R.argmax_rows(y)[:, 0]) == [0, 2, 0]
    table = rng.standard_normal((11, 4)).astype(np.float32)
    ids = np.array([10, 0, 3, 3], dtype=np.uint32)
    assert np.array_equal(R.embed(table, ids), table[ids])

"""Generates tests/golden/ref_cuda_*.npz by running the reference's OWN CUDA
operators (oracle/_ref/libref_gqa_gpu.so, compiled from the reference tree by
`make -C oracle ref`) on a GPU.  Run from the repository root on a B200:

    python tests/golden/make_golden.py [output_dir]

Small cases store their inputs; the TinyLLaMA-size layer (BASELINE config 1)
stores the seed that regenerates them with `inputs_from_seed` below and a
strided sub-sample of the output.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import cref  # noqa: E402


def layer_inputs_from_seed(seed, S, hidden, Hq, Hkv, D):
    """x ~ N(0,1); Wq, Wo, Wk, Wv ~ N(0, 0.02) (BASELINE config 1), fp32."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((S, hidden), dtype=np.float32)
    wq = (rng.standard_normal((hidden, Hq * D)) * 0.02).astype(np.float32)
    wk = (rng.standard_normal((hidden, Hkv * D)) * 0.02).astype(np.float32)
    wv = (rng.standard_normal((hidden, Hkv * D)) * 0.02).astype(np.float32)
    wo = (rng.standard_normal((Hq * D, hidden)) * 0.02).astype(np.float32)
    return x, wq, wk, wv, wo


def main(out_dir):
    os.makedirs(out_dir, exist_ok=True)
    inv = {D: cref.gpu_inv_freq(D) for D in (32, 64)}
    rng = np.random.default_rng(2024)
    n = 0

    def save(name, **kw):
        nonlocal n
        np.savez_compressed(os.path.join(out_dir, f"ref_cuda_{name}.npz"), **kw)
        n += 1

    for D, rows, cols, off in ((64, 8, 128, 0), (64, 4, 128, 2040), (32, 4, 64, 0)):
        x = rng.standard_normal((rows, cols), dtype=np.float32)
        save(f"rope_d{D}_off{off}", kind="rope", x=x, out=cref.gpu_rope(x, D, 10000.0, off), D=D, Hq=cols // D,
             Hkv=cols // D, offset=off, causal=1, inv_freq=inv[D])
    for S, Hq, Hkv, D, off, causal in ((4, 4, 2, 32, 0, 1), (33, 8, 2, 64, 3, 1), (20, 4, 4, 32, 0, 0),
                                       (40, 8, 1, 64, 0, 1)):
        q = rng.standard_normal((S, Hq * D), dtype=np.float32)
        k = rng.standard_normal((S, Hkv * D), dtype=np.float32)
        v = rng.standard_normal((S, Hkv * D), dtype=np.float32)
        out = cref.gpu_attention_core(q, k, v, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, position_offset=off,
                                      causal=bool(causal))
        save(f"core_s{S}_h{Hq}_{Hkv}_d{D}_off{off}_c{causal}", kind="core", q=q, k=k, v=v, out=out, Hq=Hq, Hkv=Hkv,
             D=D, offset=off, causal=causal, inv_freq=inv[D])
    # op_rmsnorm (src/ops/op_rmsnorm.cuh): TinyLLaMA hidden size, a width that is not a multiple of the kernel's
    # 256 threads, and a single column
    for rows, hidden in ((6, 2048), (5, 300), (3, 1)):
        x = (rng.standard_normal((rows, hidden), dtype=np.float32) * 2).astype(np.float32)
        w = (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
        save(f"rmsnorm_r{rows}_h{hidden}", kind="rmsnorm", x=x, w=w, eps=np.float32(1e-6),
             out=cref.gpu_rmsnorm(x, w, 1e-6))
    # op_argmax (src/ops/op_reduction.cuh): random rows, ties, NaN at and after element 0, a row of -inf
    x = rng.standard_normal((12, 97), dtype=np.float32)
    x[1, [4, 40, 90]] = 7.0
    x[2, 10] = np.nan
    x[3, 0] = np.nan
    x[4, :] = -np.inf
    x[5, 96] = 9.0
    save("argmax_r12_c97", kind="argmax", x=x, out=cref.gpu_argmax(x))
    # the reference's own decoder-layer test shape (test_llama.py:142-165): hidden 128, 4 heads / 2 KV heads
    S, hidden, Hq, Hkv, D = 4, 128, 4, 2, 32
    x, wq, wk, wv, wo = layer_inputs_from_seed(7, S, hidden, Hq, Hkv, D)
    out = cref.gpu_gqa_layer(x, wq, wk, wv, wo, num_heads=Hq, num_kv_heads=Hkv, head_dim=D)
    save("layer_small", kind="layer", x=x, wq=wq, wk=wk, wv=wv, wo=wo, out=out, Hq=Hq, Hkv=Hkv, D=D, offset=0,
         causal=1, inv_freq=inv[D])
    # BASELINE config 1: S=128, hidden 2048, 32q/4kv, D=64 — seed + sub-sampled output
    S, hidden, Hq, Hkv, D = 128, 2048, 32, 4, 64
    x, wq, wk, wv, wo = layer_inputs_from_seed(0, S, hidden, Hq, Hkv, D)
    out = cref.gpu_gqa_layer(x, wq, wk, wv, wo, num_heads=Hq, num_kv_heads=Hkv, head_dim=D)
    save("layer_config1", kind="layer_seeded", seed=0, S=S, hidden=hidden, out_sub=out[::4, ::16], sub_rows=4,
         sub_cols=16, out_absmax=np.abs(out).max(), Hq=Hq, Hkv=Hkv, D=D, offset=0, causal=1, inv_freq=inv[D])
    print(f"wrote {n} fixtures to {out_dir}")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden"))

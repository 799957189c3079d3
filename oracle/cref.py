"""ctypes front-end to the plain-C restatement (oracle/ref_attention.c) and,
when built, to the driver around the reference's own CUDA operators
(oracle/ref_harness.cu -> oracle/_ref/libref_gqa_gpu.so).

TEST INFRASTRUCTURE ONLY — see the header of ref_attention.c.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_CPU_SO = os.path.join(_HERE, "_build", "libref_attention.so")
_GPU_SO = os.path.join(_HERE, "_ref", "libref_gqa_gpu.so")

_fp = C.POINTER(C.c_float)


def _p(a: np.ndarray):
    return a.ctypes.data_as(_fp)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def build_cpu(force: bool = False) -> str:
    """Compile the C restatement (gcc, a second or two)."""
    if force or not os.path.exists(_CPU_SO) or os.path.getmtime(_CPU_SO) < os.path.getmtime(
            os.path.join(_HERE, "ref_attention.c")):
        subprocess.check_call(["make", "-C", _HERE, "-s", "_build/libref_attention.so"])
    return _CPU_SO


_cpu = None


def cpu():
    global _cpu
    if _cpu is None:
        _cpu = C.CDLL(build_cpu())
        _cpu.ref_num_threads.restype = C.c_int
    return _cpu


def num_threads() -> int:
    return int(cpu().ref_num_threads())


def set_num_threads(n: int) -> None:
    cpu().ref_set_num_threads(C.c_int(n))


def inv_freq(head_dim: int, theta: float = 10000.0) -> np.ndarray:
    out = np.empty(head_dim // 2, dtype=np.float32)
    cpu().ref_rope_inv_freq(C.c_int(head_dim), C.c_float(theta), _p(out))
    return out


def _tab(t):
    if t is None:
        return None, None
    t = _f32(t)
    return t, _p(t)


def rope(x, head_dim=64, theta=10000.0, position_offset=0, inv_freq=None):
    x = _f32(x)
    out = np.empty_like(x)
    keep, tp = _tab(inv_freq)
    cpu().ref_rope_f32(_p(x), C.c_int(x.shape[0]), C.c_int(x.shape[1]), C.c_int(head_dim), C.c_float(theta),
                       C.c_int(position_offset), tp, _p(out))
    return out


def rmsnorm(x, w, eps=1e-6):
    """Bit-faithful restatement of op_rmsnorm (src/ops/op_rmsnorm.cuh:8-53)."""
    x, w = _f32(x), _f32(w).reshape(-1)
    out = np.empty_like(x)
    cpu().ref_rmsnorm_f32(_p(x), _p(w), C.c_int(x.shape[0]), C.c_int(x.shape[1]), C.c_float(eps), _p(out))
    return out


def add_rmsnorm(x, residual, w, eps=1e-6):
    """s = x + residual (fp32), y = rmsnorm(s): returns (s, y)."""
    x, residual, w = _f32(x), _f32(residual), _f32(w).reshape(-1)
    s, y = np.empty_like(x), np.empty_like(x)
    cpu().ref_add_rmsnorm_f32(_p(x), _p(residual), _p(w), C.c_int(x.shape[0]), C.c_int(x.shape[1]), C.c_float(eps),
                              _p(s), _p(y))
    return s, y


def softmax(x, causal=False, seq_offset=0):
    x = _f32(x)
    out = np.empty_like(x)
    cpu().ref_softmax_f32(_p(x), C.c_int(x.shape[0]), C.c_int(x.shape[1]), C.c_int(int(causal)),
                          C.c_int(seq_offset), _p(out))
    return out


def attention_collapsed(q, k, v, *, num_heads, num_kv_heads, head_dim, theta=10000.0, position_offset=0,
                        causal=True, inv_freq=None):
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty_like(q)
    keep, tp = _tab(inv_freq)
    rc = cpu().ref_attention_collapsed_f32(_p(q), _p(k), _p(v), C.c_int(q.shape[0]), C.c_int(num_heads),
                                           C.c_int(num_kv_heads), C.c_int(head_dim), C.c_float(theta),
                                           C.c_int(position_offset), C.c_int(int(causal)), tp, _p(out))
    assert rc == 0
    return out


def gqa_layer(x, wq, wk, wv, wo, *, num_heads, num_kv_heads, head_dim, theta=10000.0, position_offset=0,
              causal=True, inv_freq=None):
    x, wq, wk, wv, wo = map(_f32, (x, wq, wk, wv, wo))
    out = np.empty((x.shape[0], wo.shape[1]), dtype=np.float32)
    keep, tp = _tab(inv_freq)
    rc = cpu().ref_gqa_layer_f32(_p(x), _p(wq), _p(wk), _p(wv), _p(wo), C.c_int(x.shape[0]), C.c_int(x.shape[1]),
                                 C.c_int(num_heads), C.c_int(num_kv_heads), C.c_int(head_dim), C.c_float(theta),
                                 C.c_int(position_offset), C.c_int(int(causal)), tp, _p(out))
    assert rc == 0
    return out


def attention_per_head(q, k, v, *, theta=10000.0, position_offset=0, causal=True, round_bf16=False,
                       inv_freq=None, batches=None, heads=None):
    """q (B,S,Hq,D), k,v (B,S,Hkv,D) float32.  `batches`/`heads` = (lo, hi)
    restrict the work (rows outside stay zero)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    out = np.zeros_like(q)
    b0, b1 = batches if batches else (0, B)
    h0, h1 = heads if heads else (0, Hq)
    keep, tp = _tab(inv_freq)
    rc = cpu().ref_attention_per_head_f32(_p(q), _p(k), _p(v), C.c_int(B), C.c_int(S), C.c_int(Hq), C.c_int(Hkv),
                                          C.c_int(D), C.c_float(theta), C.c_int(position_offset),
                                          C.c_int(int(causal)), C.c_int(int(round_bf16)), tp, C.c_int(b0),
                                          C.c_int(b1), C.c_int(h0), C.c_int(h1), _p(out))
    assert rc == 0
    return out


def decode_paged(q_rot, pool_bits, page_table, seq_lens, *, num_heads, num_kv_heads, head_dim, seqs=None):
    """q_rot (B, Hq*D) float32 already rotated; pool_bits uint16
    (num_pages, Hkv, 2, 16, D).  Returns out (B, Hq*D), lse (B, Hq)."""
    q = _f32(q_rot)
    pool = np.ascontiguousarray(pool_bits, dtype=np.uint16)
    pt = np.ascontiguousarray(page_table, dtype=np.int32)
    sl = np.ascontiguousarray(seq_lens, dtype=np.int32)
    B = q.shape[0]
    out = np.zeros((B, num_heads * head_dim), dtype=np.float32)
    lse = np.full((B, num_heads), -np.inf, dtype=np.float32)
    s0, s1 = seqs if seqs else (0, B)
    rc = cpu().ref_decode_paged_f32(_p(q), pool.ctypes.data_as(C.POINTER(C.c_uint16)),
                                    pt.ctypes.data_as(C.POINTER(C.c_int32)), C.c_int(pt.shape[1]),
                                    sl.ctypes.data_as(C.POINTER(C.c_int32)), C.c_int(num_heads),
                                    C.c_int(num_kv_heads), C.c_int(head_dim), C.c_int(s0), C.c_int(s1), _p(out),
                                    _p(lse))
    assert rc == 0
    return out, lse


# ---------------------------------------------------------------------------
# The reference's own CUDA operators (needs a GPU and oracle/_ref built)
# ---------------------------------------------------------------------------
def gpu_available() -> bool:
    return os.path.exists(_GPU_SO)


_gpu = None


def gpu():
    global _gpu
    if _gpu is None:
        _gpu = C.CDLL(_GPU_SO)
        _gpu.refgpu_last_error.restype = C.c_char_p
    return _gpu


def _gcheck(rc):
    if rc != 0:
        raise RuntimeError(gpu().refgpu_last_error().decode())


def gpu_inv_freq(head_dim, theta=10000.0):
    out = np.empty(head_dim // 2, dtype=np.float32)
    _gcheck(gpu().refgpu_inv_freq(C.c_int(head_dim), C.c_float(theta), _p(out)))
    return out


def gpu_rope(x, head_dim=64, theta=10000.0, position_offset=0):
    x = _f32(x)
    out = np.empty_like(x)
    _gcheck(gpu().refgpu_rope(_p(x), C.c_int(x.shape[0]), C.c_int(x.shape[1]), C.c_int(head_dim),
                              C.c_float(theta), C.c_int(position_offset), _p(out)))
    return out


def gpu_argmax(x):
    """The reference's own op_argmax on the GPU (needs oracle/_ref): (rows, 1) uint32."""
    x = _f32(x)
    out = np.zeros((x.shape[0], 1), dtype=np.uint32)
    _gcheck(gpu().refgpu_argmax(_p(x), C.c_int(x.shape[0]), C.c_int(x.shape[1]),
                                out.ctypes.data_as(C.POINTER(C.c_uint32))))
    return out


def gpu_rmsnorm(x, w, eps=1e-6):
    """The reference's own op_rmsnorm on the GPU (needs oracle/_ref)."""
    x, w = _f32(x), _f32(w).reshape(-1)
    out = np.empty_like(x)
    _gcheck(gpu().refgpu_rmsnorm(_p(x), _p(w), C.c_int(x.shape[0]), C.c_int(x.shape[1]), C.c_float(eps), _p(out)))
    return out


def gpu_attention_core(q, k, v, *, num_heads, num_kv_heads, head_dim, theta=10000.0, position_offset=0,
                       causal=True, apply_rope=True):
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty_like(q)
    _gcheck(gpu().refgpu_attention_core(_p(q), _p(k), _p(v), C.c_int(q.shape[0]), C.c_int(num_heads),
                                        C.c_int(num_kv_heads), C.c_int(head_dim), C.c_float(theta),
                                        C.c_int(position_offset), C.c_int(int(causal)), C.c_int(int(apply_rope)),
                                        _p(out)))
    return out


def gpu_gqa_layer(x, wq, wk, wv, wo, *, num_heads, num_kv_heads, head_dim, theta=10000.0, position_offset=0,
                  causal=True, time_iters=0, warmup=3):
    x, wq, wk, wv, wo = map(_f32, (x, wq, wk, wv, wo))
    out = np.empty((x.shape[0], wo.shape[1]), dtype=np.float32)
    ms = C.c_float(0)
    _gcheck(gpu().refgpu_gqa_layer(_p(x), _p(wq), _p(wk), _p(wv), _p(wo), C.c_int(x.shape[0]), C.c_int(x.shape[1]),
                                   C.c_int(num_heads), C.c_int(num_kv_heads), C.c_int(head_dim), C.c_float(theta),
                                   C.c_int(position_offset), C.c_int(int(causal)), _p(out), C.c_int(warmup),
                                   C.c_int(time_iters), C.byref(ms) if time_iters else None))
    return (out, float(ms.value)) if time_iters else out

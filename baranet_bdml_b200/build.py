"""Builds libbn_attn.so (the C-ABI attention module) in-tree with nvcc for
sm_100a.  Usage: python -m baranet_bdml_b200.build [--force] [--verbose]"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libbn_attn.so")
SOURCES = ["api.cu", "tma.cu", "attn_f32.cu", "rmsnorm.cu", "embed_argmax.cu", "kv_cache.cu", "attn_decode.cu", "attn_prefill_sm100.cu", "gemm_bf16_sm100.cu", "gemm_skinny.cu", "exchange.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared",
              "-I" + os.path.join(ROOT, "include"), "-I" + CSRC]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, "include", "bn_attn.h"), __file__]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, extra_flags=(), out: str = LIB) -> str:
    if out == LIB and not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
          list(extra_flags) + [os.path.join(CSRC, s) for s in SOURCES] + ["-o", out]
    env = dict(os.environ)
    # the image exports CC/CXX wrappers that lack some spec files; nvcc should use the system g++
    env.pop("CC", None)
    env.pop("CXX", None)
    res = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libbn_attn.so")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

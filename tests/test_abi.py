"""The C-ABI library loads and exports every symbol include/bn_attn.h declares;
argument errors come back as status codes (no GPU needed)."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "bn_attn.h")).read()
    return sorted(set(re.findall(r"^BN_API [\w\s\*]+?\b(bn_\w+)\(", text, flags=re.M)))


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    for must in ("bn_last_error", "bn_mm_f32", "bn_rope_f32", "bn_attn_prefill_f32", "bn_attn_prefill_bf16",
                 "bn_attn_prefill_bf16_workspace_bytes", "bn_kv_append", "bn_attn_decode_paged",
                 "bn_attn_decode_workspace_bytes", "bn_attn_lse_combine", "bn_workspace_status"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    from baranet_bdml_b200 import _lib
    for name in declared_symbols():
        assert hasattr(lib, name), name
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"


def test_bad_arguments_return_status_codes(lib):
    from baranet_bdml_b200 import _lib
    assert lib.bn_mm_f32(None, 0, 0, None, 0, 0, None, 0, 0, 1, 1, 1, None) == _lib.BN_ERR_INVALID_ARG
    assert "null pointer" in _lib.last_error()
    assert lib.bn_attn_prefill_bf16_workspace_bytes(1, 128, 8, 2, 32) == 0      # head_dim 32 unsupported
    assert lib.bn_attn_prefill_bf16_workspace_bytes(8, 2048, 32, 4, 64) > 8 * 2048 * 4 * 64 * 2
    assert lib.bn_attn_decode_workspace_bytes(64, 32, 4, 64, 4096, 100) == 0     # chunk not a multiple of 128
    assert lib.bn_attn_decode_workspace_bytes(64, 32, 4, 64, 4096, 0) > 0
    with pytest.raises(RuntimeError, match="null pointer"):
        _lib.check(lib.bn_rope_f32(None, 0, 0, None, 0, 0, 1, 64, 64, 10000.0, 0, None))


def test_missing_library_fails_loudly(monkeypatch):
    from baranet_bdml_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libbn_attn.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()


def test_host_mirror_shapes_without_gpu():
    """TensorF view arithmetic (transpose / slice / getitem) follows Tensor<T> (src/utils/tensor.cuh:133-177)."""
    import numpy as np
    from baranet_bdml_b200.tensor import TensorF
    t = TensorF(6, 8, is_cuda=False)
    a = np.arange(48, dtype=np.float32).reshape(6, 8)
    t.copy_from_numpy(a)
    assert t.shape == (6, 8) and not t.is_cuda
    assert np.array_equal(t.T.to_numpy(), a.T)
    assert np.array_equal(t[1:4, 2:].to_numpy(), a[1:4, 2:])
    assert np.array_equal(t.T[3, :].to_numpy(), a.T[3:4, :])
    assert np.array_equal(t[-1].to_numpy(), a[-1:])
    with pytest.raises(RuntimeError, match="Slice index out of range"):
        t.slice(0, 7, 0, 8)
    with pytest.raises(IndexError):
        t[::2]
    with pytest.raises(RuntimeError, match="only GPU implementation available"):
        t @ t.T


C_CALLER = r"""
#include <stdio.h>
#include <string.h>
#include "bn_attn.h"
int main(void) {
    /* a caller that has nothing but the header: statuses, the size queries and argument checks need no GPU */
    if (bn_version() < 100) return 1;
    if (bn_mm_f32(NULL, 0, 0, NULL, 0, 0, NULL, 0, 0, 1, 1, 1, NULL) != BN_ERR_INVALID_ARG) return 2;
    if (strstr(bn_last_error(), "null pointer") == NULL) return 3;
    if (bn_attn_prefill_bf16_workspace_bytes(8, 2048, 32, 4, 64) == 0) return 4;
    if (bn_attn_decode_workspace_bytes(64, 32, 4, 64, 4096, 0) == 0) return 5;
    printf("ok %d\n", bn_version());
    return 0;
}
"""


@pytest.mark.parametrize("compiler,ext,std", [("gcc", ".c", "-std=c99"), ("g++", ".cpp", "-std=c++11")])
def test_header_serves_a_plain_c_and_a_cpp_caller(lib, tmp_path, compiler, ext, std):
    """include/bn_attn.h compiled by a C and by a C++ compiler from outside the library (the position of the
    reference's C++ layer, src/llama/llama_layers.hpp:57-113), linked against the built library and run."""
    import subprocess
    from baranet_bdml_b200 import _lib
    src = tmp_path / ("caller" + ext)
    src.write_text(C_CALLER)
    exe = tmp_path / "caller"
    libdir = os.path.dirname(_lib.LIB_PATH)
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    subprocess.run([compiler, std, "-Wall", "-Wextra", "-Werror", "-pedantic", "-I" + os.path.join(ROOT, "include"),
                    str(src), "-o", str(exe), "-L" + libdir, "-l:" + os.path.basename(_lib.LIB_PATH),
                    "-Wl,-rpath," + libdir], check=True, env=env, capture_output=True, text=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert res.returncode == 0, (res.returncode, res.stdout, res.stderr)
    assert res.stdout.startswith("ok")

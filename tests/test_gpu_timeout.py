"""The bounded device-side waits: a wait that cannot be satisfied ends with a status, not with a hung GPU.

The failure is made by a barrier that nothing arrives at (bn_selftest_wait_timeout, 1 ms limit): the kernel's wait
gives up, stores BN_ERR_TIMEOUT at the head of the scratch buffer and returns.  Afterwards the same buffer, zeroed
again as the header says, serves an ordinary launch."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_reports_timeout_and_the_scratch_recovers(lib):
    from baranet_bdml_b200 import _lib, ops
    B, S, Hq, Hkv, D = 1, 256, 8, 2, 64
    ws = ops.prefill_workspace(B, S, Hq, Hkv, D)
    q = torch.randn((B, S, Hq, D), device="cuda").to(torch.bfloat16)
    k = torch.randn((B, S, Hkv, D), device="cuda").to(torch.bfloat16)
    v = torch.randn((B, S, Hkv, D), device="cuda").to(torch.bfloat16)
    want = ops.attn_prefill_bf16(q, k, v, workspace=ws).clone()
    torch.cuda.synchronize()
    ws.status()

    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    _lib.check(lib.bn_selftest_wait_timeout(ws.ptr, 1000, torch.cuda.current_stream().cuda_stream))
    t1.record()
    torch.cuda.synchronize()
    assert 0.5 <= t0.elapsed_time(t1) <= 200.0            # it waited about its limit, and it came back
    with pytest.raises(RuntimeError, match="bounded device-side wait ran out"):
        ws.status()
    assert lib.bn_workspace_status(ws.ptr, None) == _lib.BN_ERR_TIMEOUT

    ws.buf.zero_()                                         # "zero-filled again before reuse"
    got = ops.attn_prefill_bf16(q, k, v, workspace=ws)
    torch.cuda.synchronize()
    ws.status()
    assert torch.equal(got, want)


def test_static_decode_scratch_status_is_clean(lib):
    from baranet_bdml_b200 import _lib
    assert lib.bn_attn_decode_paged_static_status(None) == _lib.BN_OK


def test_selftest_rejects_bad_limits(lib):
    from baranet_bdml_b200 import _lib
    buf = torch.zeros(64, dtype=torch.int32, device="cuda")
    assert lib.bn_selftest_wait_timeout(buf.data_ptr(), 0, None) == _lib.BN_ERR_INVALID_ARG
    assert lib.bn_selftest_wait_timeout(None, 10, None) == _lib.BN_ERR_INVALID_ARG

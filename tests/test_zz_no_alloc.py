"""The allocation-free decode entry point (bn_attn_decode_paged_static) against the regular one.

Some callers of this library cannot allocate device memory when they call it — a plugin living inside another
engine's fixed memory plan, or a latency-critical loop that must stay away from cudaMalloc — so they cannot give
bn_attn_decode_paged its scratch buffer.  The static variant keeps that scratch inside the library.  This test calls
both through the C ABI on the same cache and checks that they agree, twice in a row (the second call finds the
scratch as the first one left it).  It is collected last, so a run that stops at the first failure has already run
everything else; it also passes on its own in a fresh process."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

Hq, Hkv, D = 32, 4, 64


def _case(seed, lens):
    from baranet_bdml_b200.kv_cache import PagedKVCache, PAGE_TOKENS
    rng = np.random.default_rng(seed)
    B = len(lens)
    pages = [(L + PAGE_TOKENS - 1) // PAGE_TOKENS for L in lens]
    max_pages = 4096 // PAGE_TOKENS
    cache = PagedKVCache(sum(pages) + 2, B, max_pages, Hkv, D)
    cache.pool.copy_(torch.randn(cache.pool.shape, device="cuda").to(torch.bfloat16))
    perm = rng.permutation(sum(pages) + 2).astype(np.int32)
    pt = np.zeros((B, max_pages), dtype=np.int32)
    at = 0
    for b in range(B):
        pt[b, :pages[b]] = perm[at:at + pages[b]]
        at += pages[b]
    cache.page_table.copy_(torch.from_numpy(pt))
    cache.seq_lens.copy_(torch.tensor(lens, dtype=torch.int32))
    q = torch.randn((B, Hq, D), device="cuda").to(torch.bfloat16)
    return cache, q


def _regular(lib, cache, q):
    from baranet_bdml_b200 import _lib
    B = q.shape[0]
    out = torch.empty((B, Hq, D), dtype=torch.float32, device="cuda")
    lse = torch.empty((B, Hq), dtype=torch.float32, device="cuda")
    ws = cache.workspace(B, Hq, 4096, 0)
    _lib.check(lib.bn_attn_decode_paged(q.data_ptr(), cache.pool.data_ptr(), cache.num_pages,
                                        cache.page_table.data_ptr(), cache.max_pages, cache.seq_lens.data_ptr(), None,
                                        None, out.data_ptr(), lse.data_ptr(), B, Hq, Hkv, D, 0.125, 10000.0, 1, 4096, 0,
                                        ws.ptr, ws.nbytes, None))
    torch.cuda.synchronize()
    return out.cpu().numpy(), lse.cpu().numpy()


def _static(lib, cache, q):
    from baranet_bdml_b200 import _lib
    B = q.shape[0]
    out = torch.empty((B, Hq, D), dtype=torch.float32, device="cuda")
    lse = torch.empty((B, Hq), dtype=torch.float32, device="cuda")
    _lib.check(lib.bn_attn_decode_paged_static(q.data_ptr(), cache.pool.data_ptr(), cache.num_pages,
                                               cache.page_table.data_ptr(), cache.max_pages,
                                               cache.seq_lens.data_ptr(), None, None, out.data_ptr(), lse.data_ptr(),
                                               B, Hq, Hkv, D, 0.125, 10000.0, 1, 4096, None))
    torch.cuda.synchronize()
    return out.cpu().numpy(), lse.cpu().numpy()


def test_static_scratch_decode_matches_regular_entry_twice(lib):
    # two different batches back to back: long sequences are cut across CTAs, so the scratch really is used
    for seed, lens in ((1, [4096, 3000, 17, 2048, 1, 4095, 1500, 777]), (2, [3500] * 16 + [64] * 8)):
        cache, q = _case(seed, lens)
        ref, ref_lse = _regular(lib, cache, q)
        got, got_lse = _static(lib, cache, q)
        assert np.isfinite(got).all()
        assert np.abs(got - ref).max() <= 1e-3
        assert np.abs(got_lse - ref_lse).max() <= 1e-3


def test_static_scratch_survives_a_growing_batch(lib):
    """The words that outlive a call (the merge tickets) must not sit where an earlier, smaller batch wrote its
    partial results: a small batch of long sequences, then the largest batch the entry accepts with long sequences
    at every index, then small again.  Every (sequence, head) of the large batch is cut across CTAs."""
    from baranet_bdml_b200 import _lib
    for seed, lens in ((11, [4096] * 8), (12, [3500] * 64), (13, [4096]), (14, [2100] * 32), (15, [4096] * 8)):
        cache, q = _case(seed, lens)
        ref, ref_lse = _regular(lib, cache, q)
        got, got_lse = _static(lib, cache, q)
        assert np.isfinite(got).all()
        assert np.abs(got - ref).max() <= 1e-3, lens[:2]
        assert np.abs(got_lse - ref_lse).max() <= 1e-3
    assert lib.bn_attn_decode_paged_static_status(None) == _lib.BN_OK


def test_one_caller_owned_scratch_serves_batches_of_any_size(lib):
    """The same rule for bn_attn_decode_paged: one buffer sized for the largest batch, zero-filled once, then used
    with a small batch, the large one and a small one again; each against a fresh buffer of its own."""
    from baranet_bdml_b200 import _lib, ops
    big = ops.Workspace(lib.bn_attn_decode_workspace_bytes(64, Hq, Hkv, D, 4096, 0))
    for seed, lens in ((21, [4096] * 4), (22, [3700] * 64), (23, [4096, 5, 3000])):
        cache, q = _case(seed, lens)
        ref, ref_lse = _regular(lib, cache, q)
        B = len(lens)
        out = torch.empty((B, Hq, D), dtype=torch.float32, device="cuda")
        lse = torch.empty((B, Hq), dtype=torch.float32, device="cuda")
        _lib.check(lib.bn_attn_decode_paged(q.data_ptr(), cache.pool.data_ptr(), cache.num_pages,
                                            cache.page_table.data_ptr(), cache.max_pages, cache.seq_lens.data_ptr(),
                                            None, None, out.data_ptr(), lse.data_ptr(), B, Hq, Hkv, D, 0.125, 10000.0,
                                            1, 4096, 0, big.ptr, big.nbytes, None))
        torch.cuda.synchronize()
        big.status()
        assert np.abs(out.cpu().numpy() - ref).max() <= 1e-3, lens[:2]
        assert np.abs(lse.cpu().numpy() - ref_lse).max() <= 1e-3


def test_static_scratch_rejects_what_does_not_fit(lib):
    from baranet_bdml_b200 import _lib
    cache, q = _case(3, [100] * 4)
    out = torch.empty((4, Hq, D), dtype=torch.float32, device="cuda")
    args = (q.data_ptr(), cache.pool.data_ptr(), cache.num_pages, cache.page_table.data_ptr(), cache.max_pages,
            cache.seq_lens.data_ptr(), None, None, out.data_ptr(), None)
    assert lib.bn_attn_decode_paged_static(*args, 4, Hq, Hkv, D, 0.125, 10000.0, 1, 8192, None) == _lib.BN_ERR_UNSUPPORTED
    assert "max_seq_len" in _lib.last_error()
    assert lib.bn_attn_decode_paged_static(*args, 65, Hq, Hkv, D, 0.125, 10000.0, 1, 4096, None) == _lib.BN_ERR_UNSUPPORTED

"""Host-side logic of the multi-GPU path on CPU: partitioning, and the exchange step of the
sequence-split decode run as two gloo ranks (the merge arithmetic comes from the oracle here;
on GPUs it is bn_attn_lse_combine)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_range_covers_everything():
    from baranet_bdml_b200.dist import shard_range
    for n in (0, 1, 7, 32, 33):
        for w in (1, 2, 4, 8):
            got = [shard_range(n, w, r) for r in range(w)]
            assert got[0][0] == 0 and got[-1][1] == n
            assert all(got[i][1] == got[i + 1][0] for i in range(w - 1))
            sizes = [b - a for a, b in got]
            assert max(sizes) - min(sizes) <= 1


def test_lpt_balances_config3_lengths():
    from baranet_bdml_b200.dist import shard_sequences_by_length
    lens = np.random.default_rng(3).integers(1024, 4097, 64)
    for w in (2, 4, 8):
        parts = shard_sequences_by_length(lens, w)
        assert sorted(i for p in parts for i in p) == list(range(64))
        loads = [int(lens[p].sum()) for p in parts]
        assert max(loads) / (sum(loads) / w) < 1.03


def test_sequence_split_ranges_are_page_aligned():
    from baranet_bdml_b200.dist import sequence_split_ranges
    for L in (262144, 1000, 17, 5):
        for w in (1, 2, 4, 8):
            r = sequence_split_ranges(L, w)
            assert r[0][0] == 0 and r[-1][1] == L
            assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
            assert all(a % 16 == 0 for a, b in r if b > a)


def _rank_main(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from baranet_bdml_b200.dist import combine_partials, sequence_split_ranges
    from oracle import ref_attention as R
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(5)      # same inputs on every rank
    L, Hq, Hkv, D = 80, 8, 2, 64        # 5 pages over 2 ranks: 3 + 2
    pool = R.round_bf16(rng.standard_normal((5, Hkv, 2, 16, D), dtype=np.float32))
    pt = np.arange(5, dtype=np.int32)[None]
    q = R.round_bf16(rng.standard_normal((1, Hq * D), dtype=np.float32))
    t0, t1 = sequence_split_ranges(L, world)[rank]
    o, l = R.decode_paged(q, pool, pt, np.array([L]), num_heads=Hq, num_kv_heads=Hkv, head_dim=D, return_lse=True,
                          token_begin=np.array([t0]), token_end=np.array([t1]))

    def merge(outs, lses):
        mo, ml = R.lse_combine(outs.numpy(), lses.numpy())
        return torch.from_numpy(mo), torch.from_numpy(ml)

    mo, ml = combine_partials(torch.from_numpy(o.reshape(Hq, D).astype(np.float32)),
                              torch.from_numpy(l.reshape(Hq).astype(np.float32)), merge=merge)
    full, full_lse = R.decode_paged(q, pool, pt, np.array([L]), num_heads=Hq, num_kv_heads=Hkv, head_dim=D,
                                    return_lse=True)
    ok = (np.abs(mo.numpy().reshape(-1) - full[0]).max() < 1e-5) and (np.abs(ml.numpy() - full_lse[0]).max() < 1e-5)
    open(os.path.join(tmp, f"rank{rank}.ok" if ok else f"rank{rank}.bad"), "w").close()
    dist.destroy_process_group()


def test_sequence_split_combine_two_gloo_ranks(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["rank0.ok", "rank1.ok"]


def _missing_rank_main(rank, world, port, tmp):
    """Rank 1 never joins the collective: rank 0's all-gather must end with an error
    after the (short) process-group timeout instead of waiting forever."""
    sys.path.insert(0, ROOT)
    import datetime
    import torch.distributed as dist
    from baranet_bdml_b200.dist import combine_partials
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    if rank == 1:
        import time
        time.sleep(6)           # leaves without taking part
        open(os.path.join(tmp, "rank1.left"), "w").close()
        os._exit(0)
    try:
        combine_partials(torch.zeros(4, 8), torch.zeros(4), merge=lambda a, b: (a[0], b[0]))
        open(os.path.join(tmp, "rank0.no_error"), "w").close()
    except Exception:
        open(os.path.join(tmp, "rank0.raised"), "w").close()
    os._exit(0)


def test_missing_rank_raises_instead_of_hanging(tmp_path):
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_missing_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert "rank0.raised" in os.listdir(tmp_path)


def _deadline_main(rank, world, port, tmp):
    """Rank 1 is late (it arrives after rank 0's own deadline): rank 0 gets ExchangeTimeout after about its
    deadline, long before the process group's timeout."""
    sys.path.insert(0, ROOT)
    import datetime
    import time
    import torch.distributed as dist
    from baranet_bdml_b200.dist import ExchangeTimeout, combine_partials
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    if rank == 1:
        time.sleep(4)
        os._exit(0)
    t0 = time.monotonic()
    try:
        combine_partials(torch.zeros(4, 8), torch.zeros(4), merge=lambda a, b: (a[0], b[0]), deadline_s=1.0)
        name = "rank0.no_error"
    except ExchangeTimeout:
        name = "rank0.deadline_%d" % int(time.monotonic() - t0 < 3.0)
    open(os.path.join(tmp, name), "w").close()
    os._exit(0)


def test_exchange_deadline_fires_before_the_group_timeout(tmp_path):
    port = 33500 + (os.getpid() % 2000)
    mp.spawn(_deadline_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert "rank0.deadline_1" in os.listdir(tmp_path)

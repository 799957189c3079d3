"""Multi-GPU partitioning of the attention path (one process per GPU,
torch.distributed for the plumbing).

The reference is single-GPU (no NCCL, MPI, streams or device selection anywhere
in its tree), so everything here is new.  The path shards without any
data-path collective except in one place:

  * prefill:     (batch, KV-head group) units are independent   -> `shard_range`
  * decode:      sequences are independent; balance by length   -> `shard_sequences_by_length`
  * long context decode: ONE sequence is cut into contiguous token ranges, one
    per GPU; each GPU produces normalised partial outputs and log-sum-exps for
    its range, and the only exchange is one all-gather of (D + 1) floats per
    (sequence, query head) followed by a local log-sum-exp merge
                                                                 -> `sequence_split_ranges`, `combine_partials`
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch


def shard_range(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced [lo, hi) of n_units for this rank (sizes differ by at most 1)."""
    base, rem = divmod(int(n_units), int(world))
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_sequences_by_length(seq_lens: Sequence[int], world: int) -> List[List[int]]:
    """Longest-processing-time greedy: sequences sorted by length, each given to the
    least-loaded rank.  Returns the sequence indices of every rank (ascending)."""
    order = sorted(range(len(seq_lens)), key=lambda i: (-int(seq_lens[i]), i))
    load = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (load[j], j))
        out[r].append(i)
        load[r] += int(seq_lens[i])
    return [sorted(x) for x in out]


def sequence_split_ranges(length: int, world: int, page_tokens: int = 16) -> List[Tuple[int, int]]:
    """Contiguous page-aligned token ranges [t0, t1), one per rank, covering [0, length)."""
    pages = (int(length) + page_tokens - 1) // page_tokens
    out = []
    for r in range(world):
        lo, hi = shard_range(pages, world, r)
        out.append((min(lo * page_tokens, length), min(hi * page_tokens, length)))
    return out


class ExchangeTimeout(RuntimeError):
    """The exchange did not complete within its deadline: a rank never arrived."""


def combine_partials(out_partial: torch.Tensor, lse_partial: torch.Tensor, group=None,
                     merge: Optional[Callable] = None, deadline_s: Optional[float] = None
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """out_partial (n, D) fp32 normalised over this rank's tokens, lse_partial (n,) fp32
    natural log (-inf when the rank holds no token of the row).  One all-gather, then every
    rank merges locally, so all ranks end with identical results.

    `merge(outs[P,n,D], lses[P,n]) -> (out, lse)` defaults to the CUDA kernel
    (bn_attn_lse_combine); CPU-only tests of the exchange pass their own.
    `deadline_s`: give up with ExchangeTimeout when the collective has not completed by then."""
    import torch.distributed as dist
    n, D = out_partial.shape
    packed = torch.cat([out_partial, lse_partial.reshape(n, 1)], dim=1).contiguous()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world > 1:
        gathered = [torch.empty_like(packed) for _ in range(world)]
        if deadline_s is None:
            dist.all_gather(gathered, packed, group=group)
        else:
            # host deadline of our own, shorter than the process group's: the collective is started without blocking
            # and polled; past the deadline the caller gets ExchangeTimeout (and should tear the group down: the
            # collective that never completed leaves it unusable)
            import time
            work = dist.all_gather(gathered, packed, group=group, async_op=True)
            t_end = time.monotonic() + float(deadline_s)
            while not work.is_completed():
                if time.monotonic() > t_end:
                    raise ExchangeTimeout(f"exchange of partial results: no completion within {deadline_s} s "
                                          f"(a rank did not arrive)")
                time.sleep(0.001)
            work.wait()
        allp = torch.stack(gathered)
    else:
        allp = packed[None]
    outs = allp[:, :, :D].contiguous()
    lses = allp[:, :, D].contiguous()
    if merge is None:
        from . import ops
        merge = ops.lse_combine
    return merge(outs, lses)


class PartialExchange:
    """The exchange step of the sequence-split decode.  The decode kernel writes its normalised partial output and
    log-sum-exp straight into `out_view` / `lse_view` (two regions of one contiguous send buffer); `combine()` merges
    every rank's buffer into `out` / `lse`, identical on all ranks.  All buffers are allocated once.

    mode "nccl" (default): one all-gather into `recv`, then bn_attn_lse_combine_strided (two launches).
    mode "peer": ONE launch, bn_exchange_combine: every rank stores its partial into every rank's exchange buffer
        over NVLink peer memory (buffers made known to each other through CUDA IPC handles, gathered here with
        torch.distributed), waits for the others with a time limit and merges.  `status()` raises if a wait ran
        out; the object is then unusable.  Falls back to "nccl" (and says so in `kind`) when the peer mapping
        cannot be set up."""

    def __init__(self, n: int, D: int, group=None, device="cuda", mode: str = "nccl", wait_us: int = 1000000):
        import torch.distributed as dist
        self.n, self.D, self.group = int(n), int(D), group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.wait_us = int(wait_us)
        self.send = torch.empty(self.n * (self.D + 1), dtype=torch.float32, device=device)
        self.recv = torch.empty(self.world * self.n * (self.D + 1), dtype=torch.float32, device=device)
        self.out_view = self.send[: self.n * self.D].view(self.n, self.D)
        self.lse_view = self.send[self.n * self.D:]
        self.out = torch.empty((self.n, self.D), dtype=torch.float32, device=device)
        self.lse = torch.empty((self.n,), dtype=torch.float32, device=device)
        self._peer = None
        self.kind = "one NCCL all-gather + merge kernel" if self.world > 1 else "none (one rank)"
        if mode == "peer":
            why = self._open_peer()
            if why is None:
                self.kind = "one kernel: peer stores over NVLink + bounded wait + merge"
            else:
                self.kind += f" (peer exchange unavailable: {why})"
        elif mode != "nccl":
            raise ValueError(f"PartialExchange: unknown mode {mode!r}")

    def _open_peer(self) -> Optional[str]:
        """None on success, else the reason (every rank takes the same decision)."""
        import ctypes as C
        import torch.distributed as dist
        from . import _lib
        lib = _lib.load()
        handle = C.c_void_p()
        ok, why = True, ""
        if lib.bn_exchange_create(self.n, self.D, self.world, self.rank, C.byref(handle)) != _lib.BN_OK:
            ok, why = False, _lib.last_error()
        mine = (C.c_char * 64)()
        if ok and self.world > 1 and lib.bn_exchange_ipc_handle(handle, mine) != _lib.BN_OK:
            ok, why = False, _lib.last_error()
        if self.world > 1:
            gathered = [None] * self.world
            dist.all_gather_object(gathered, (ok, why, bytes(mine)), group=self.group)
            bad = [g for g in gathered if not g[0]]
            if bad:
                if handle:
                    lib.bn_exchange_destroy(handle)
                return bad[0][1]
            blob = b"".join(g[2] for g in gathered)
            rc = lib.bn_exchange_open_peers(handle, blob, 0)
            results = [None] * self.world
            dist.all_gather_object(results, (rc, _lib.last_error() if rc else ""), group=self.group)
            bad = [r for r in results if r[0] != _lib.BN_OK]
            if bad:
                lib.bn_exchange_destroy(handle)
                return bad[0][1]
        else:
            if not ok:
                return why
            if lib.bn_exchange_open_peers(handle, None, 1) != _lib.BN_OK:
                why = _lib.last_error()
                lib.bn_exchange_destroy(handle)
                return why
        self._peer = handle
        return None

    def combine(self) -> Tuple[torch.Tensor, torch.Tensor]:
        import torch.distributed as dist
        from . import _lib
        stream = torch.cuda.current_stream().cuda_stream
        if self._peer is not None:
            _lib.check(_lib.load().bn_exchange_combine(self._peer, self.send.data_ptr(), self.out.data_ptr(),
                                                       self.lse.data_ptr(), self.wait_us, stream))
            return self.out, self.lse
        src = self.send
        if self.world > 1:
            dist.all_gather_into_tensor(self.recv, self.send, group=self.group)
            src = self.recv
        stride = self.n * (self.D + 1)
        _lib.check(_lib.load().bn_attn_lse_combine_strided(
            src.data_ptr(), stride, src.data_ptr() + 4 * self.n * self.D, stride, self.world, self.n, self.D,
            self.out.data_ptr(), None, self.lse.data_ptr(), stream))
        return self.out, self.lse

    def status(self) -> None:
        """Raises if a bounded wait of the peer exchange ran out (a rank never delivered)."""
        if self._peer is not None:
            from . import _lib
            _lib.check(_lib.load().bn_exchange_status(self._peer, torch.cuda.current_stream().cuda_stream))

    def close(self) -> None:
        if self._peer is not None:
            from . import _lib
            _lib.load().bn_exchange_destroy(self._peer)
            self._peer = None

"""Functional front-end of the bf16 kernels on torch CUDA tensors (torch is
used for device memory and streams only; all arithmetic is in libbn_attn.so).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, dtype, what: str):
    if not t.is_cuda:
        raise RuntimeError(f"{what}: only GPU implementation available")
    if t.dtype != dtype or not t.is_contiguous():
        raise RuntimeError(f"{what}: expected a contiguous {dtype} tensor")


class Workspace:
    """A caller-owned scratch buffer (256-byte aligned, zero-filled once)."""

    def __init__(self, nbytes: int, device=None):
        self.buf = torch.zeros(max(int(nbytes), 256) + 256, dtype=torch.uint8, device=device or "cuda")
        self.ptr = (self.buf.data_ptr() + 255) // 256 * 256
        self.nbytes = self.buf.numel() - (self.ptr - self.buf.data_ptr())

    def status(self) -> None:
        """Raises if a kernel that used this buffer gave up on a bounded wait."""
        _lib.check(_lib.load().bn_workspace_status(self.ptr, _stream()))


def prefill_workspace(B: int, S: int, Hq: int, Hkv: int, D: int = 64, device=None) -> Workspace:
    n = _lib.load().bn_attn_prefill_bf16_workspace_bytes(B, S, Hq, Hkv, D)
    if n == 0:
        raise RuntimeError(f"bn_attn_prefill_bf16: unsupported shape B={B} S={S} Hq={Hq} Hkv={Hkv} D={D}")
    return Workspace(n, device)


def attn_prefill_bf16(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: Optional[float] = None,
                      theta: float = 10000.0, position_offset: int = 0, causal: bool = True,
                      out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None,
                      workspace: Optional[Workspace] = None, reuse_rotated_k: bool = False,
                      single_tile_kernel: bool = False) -> torch.Tensor:
    """q (B,S,Hq,D), k,v (B,S,Hkv,D) bf16, q/k pre-RoPE -> out (B,S,Hq,D) bf16.
    `reuse_rotated_k`: the workspace still holds the rotated K of an earlier
    call on the same k and position_offset (skips the rotation launch).
    `single_tile_kernel` selects the simpler kernel variant kept for comparison."""
    if k is None and not reuse_rotated_k:
        raise RuntimeError("attn_prefill_bf16: k may only be omitted when the workspace already holds the rotated K")
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        if t is not None:
            _need(t, torch.bfloat16, f"attn_prefill_bf16({n})")
    B, S, Hq, D = q.shape
    Hkv = v.shape[2]
    if v.shape != (B, S, Hkv, D) or (k is not None and k.shape != v.shape):
        raise RuntimeError("Attention: hidden size mismatch")
    if out is None:
        out = torch.empty_like(q)
    if workspace is None:
        workspace = prefill_workspace(B, S, Hq, Hkv, D, q.device)
    if scale is None:
        scale = 1.0 / (D ** 0.5)
    _lib.check(_lib.load().bn_attn_prefill_bf16(
        q.data_ptr(), k.data_ptr() if k is not None else None, v.data_ptr(), out.data_ptr(),
        lse.data_ptr() if lse is not None else None,
        B, S, Hq, Hkv, D, float(scale), float(theta), int(position_offset), int(bool(causal)),
        (0x100 if reuse_rotated_k else 0) | (0x200 if single_tile_kernel else 0),
        workspace.ptr, workspace.nbytes, _stream()))
    return out


def prefill_table(workspace: Workspace, B: int, S: int, Hkv: int, D: int = 64, theta: float = 10000.0,
                  position_offset: int = 0) -> None:
    """Writes the cos/sin table of positions position_offset .. position_offset + S - 1 into a prefill scratch buffer
    (what the K-rotation launch of attn_prefill_bf16 does on the side), for use with gemm_qkv_rope_bf16."""
    _lib.check(_lib.load().bn_attn_prefill_bf16_table(B, S, Hkv, D, float(theta), int(position_offset), workspace.ptr,
                                                      workspace.nbytes, _stream()))


def gemm_qkv_rope_bf16(x: torch.Tensor, wqkv_t: torch.Tensor, B: int, S: int, Hq: int, Hkv: int, D: int,
                       workspace: Workspace, *, position_offset: int = 0, cache=None,
                       error_word: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """The layer's q, k and v projections as one GEMM: x (B*S, hidden) bf16, wqkv_t ((Hq + 2 Hkv) D, hidden) bf16
    (rows of Wq^T, Wk^T, Wv^T).  Returns q (B, S, Hq, D) as projected and v (B, S, Hkv, D); the rotated K and its
    norms are left in `workspace` (whose table must be current: prefill_table) for
    attn_prefill_bf16(q, None, v, workspace=workspace, reuse_rotated_k=True); with `cache` (a PagedKVCache whose
    sequences are the B rows) rotated K and V are also appended at positions position_offset .. + S - 1."""
    _need(x, torch.bfloat16, "gemm_qkv_rope_bf16(x)")
    _need(wqkv_t, torch.bfloat16, "gemm_qkv_rope_bf16(wqkv_t)")
    hidden = x.shape[1]
    if x.shape[0] != B * S or wqkv_t.shape != ((Hq + 2 * Hkv) * D, hidden):
        raise RuntimeError(f"MatMul: inner dimensions mismatch {tuple(x.shape)} x {tuple(wqkv_t.shape)}^T")
    q = torch.empty((B, S, Hq, D), dtype=torch.bfloat16, device=x.device)
    v = torch.empty((B, S, Hkv, D), dtype=torch.bfloat16, device=x.device)
    pool = pages = None
    n_pages = max_pages = 0
    if cache is not None:
        pool, pages, n_pages, max_pages = cache.pool.data_ptr(), cache.page_table.data_ptr(), cache.num_pages, cache.max_pages
    _lib.check(_lib.load().bn_gemm_qkv_rope_bf16(
        x.data_ptr(), wqkv_t.data_ptr(), q.data_ptr(), v.data_ptr(), B, S, hidden, Hq, Hkv, D, int(position_offset),
        workspace.ptr, workspace.nbytes, pool, n_pages, pages, max_pages,
        _gemm_error_ptr(x.device, error_word), _stream()))
    return q, v


_gemm_err = {}


def _gemm_error_ptr(device, given: Optional[torch.Tensor]):
    """The error word a tcgen05 GEMM launch reports a bounded wait that ran out into: the caller's, else one int32 per
    device that lives as long as the process (`gemm_status` reads it).  None only while a stream capture is the first
    thing that asks for it (no allocation inside a capture)."""
    if given is not None:
        return given.data_ptr()
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    word = _gemm_err.get(key)
    if word is None:
        if torch.cuda.is_current_stream_capturing():
            return None
        word = _gemm_err[key] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
    return word.data_ptr()


def gemm_status(device=None) -> None:
    """Raises if any GEMM launched without an error word of its own gave up a bounded wait on this device since the
    last call (its output is then garbage); clears the word.  Synchronises."""
    key = torch.cuda.current_device() if device is None else torch.device(device).index
    word = _gemm_err.get(key)
    if word is not None:
        code = int(word.item())
        if code != 0:
            word.zero_()
            raise RuntimeError(f"a projection GEMM reported error {code} (a bounded wait ran out)")


def gemm_bf16_nt(a: torch.Tensor, bt: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                 error_word: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a (M,K) bf16 @ bt (N,K)^T bf16 -> (M,N) bf16, fp32 accumulation: the layer's projections `x @ W` with the weight
    stored as (out_features, in_features)."""
    _need(a, torch.bfloat16, "gemm_bf16_nt(a)")
    _need(bt, torch.bfloat16, "gemm_bf16_nt(bt)")
    if a.dim() != 2 or bt.dim() != 2 or a.shape[1] != bt.shape[1]:
        raise RuntimeError(f"MatMul: inner dimensions mismatch {tuple(a.shape)} x {tuple(bt.shape)}^T")
    M, K = a.shape
    N = bt.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    _need(out, torch.bfloat16, "gemm_bf16_nt(out)")
    _lib.check(_lib.load().bn_gemm_bf16_nt(a.data_ptr(), bt.data_ptr(), out.data_ptr(), M, N, K,
                                           _gemm_error_ptr(a.device, error_word), _stream()))
    return out


_small_m_ws = {}


def gemm_bf16_nt_small_m(a: torch.Tensor, bt: torch.Tensor, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a (M,K) @ bt (N,K)^T for few rows (a decode step: one token per sequence): the weight stream is spread over
    all SMs (64-wide N tiles, K split, partial sums added in a fixed order).  The fp32 scratch is kept per
    (device, size) and reused by later calls on the same stream."""
    _need(a, torch.bfloat16, "gemm_bf16_nt_small_m(a)")
    _need(bt, torch.bfloat16, "gemm_bf16_nt_small_m(bt)")
    if a.dim() != 2 or bt.dim() != 2 or a.shape[1] != bt.shape[1]:
        raise RuntimeError(f"MatMul: inner dimensions mismatch {tuple(a.shape)} x {tuple(bt.shape)}^T")
    M, K = a.shape
    N = bt.shape[0]
    lib = _lib.load()
    n = int(lib.bn_gemm_bf16_nt_small_m_workspace_bytes(M, N, K))
    key = (a.device, n)
    ws = _small_m_ws.get(key)
    if ws is None:
        ws = _small_m_ws[key] = torch.empty(max(n, 16), dtype=torch.uint8, device=a.device)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    _need(out, torch.bfloat16, "gemm_bf16_nt_small_m(out)")
    _lib.check(lib.bn_gemm_bf16_nt_small_m(a.data_ptr(), bt.data_ptr(), out.data_ptr(), M, N, K, ws.data_ptr(), n,
                                           _gemm_error_ptr(a.device, None), _stream()))
    return out


def skinny_ok(rows: int, n_out: int, k: int) -> bool:
    """Shapes the weight-streaming kernel for at most 16 rows takes."""
    return 0 < rows <= 16 and n_out % 8 == 0 and k % 256 == 0 and 0 < k <= 8192


def gemm_bf16_nt_skinny(x: torch.Tensor, weight_t: torch.Tensor, splits: Optional[Tuple[int, ...]] = None):
    """x (rows <= 16, in) @ weight_t (out, in)^T by streaming the weight through all SMs (warp-level MMAs whose M = 16
    is the whole batch).  `splits` = sizes of up to three column ranges that go to separate output tensors (the q, k, v
    projections over the concatenated weight); returns one tensor, or a tuple with `splits`."""
    _need(x, torch.bfloat16, "gemm_bf16_nt_skinny(x)")
    _need(weight_t, torch.bfloat16, "gemm_bf16_nt_skinny(weight_t)")
    M, K = x.shape
    N = weight_t.shape[0]
    if weight_t.shape[1] != K:
        raise RuntimeError(f"MatMul: inner dimensions mismatch {tuple(x.shape)} x {tuple(weight_t.shape)}^T")
    sizes = list(splits) if splits else [N]
    if sum(sizes) != N or not 1 <= len(sizes) <= 3:
        raise RuntimeError("gemm_bf16_nt_skinny: the column ranges must add up to the weight's rows (at most three)")
    outs = [torch.empty((M, n), dtype=torch.bfloat16, device=x.device) for n in sizes]
    ptrs = [o.data_ptr() for o in outs] + [None] * (3 - len(outs))
    n0, n1 = sizes[0], (sizes[1] if len(sizes) > 1 else 0)
    _lib.check(_lib.load().bn_gemm_bf16_nt_skinny(x.data_ptr(), weight_t.data_ptr(), M, N, K, ptrs[0], n0, ptrs[1], n1,
                                                  ptrs[2], _stream()))
    return tuple(outs) if splits else outs[0]


def gemm_qkv_append_bf16_skinny(x: torch.Tensor, wqkv_t: torch.Tensor, cache, seq_ids: torch.Tensor,
                                positions: torch.Tensor, num_heads: int) -> torch.Tensor:
    """The q, k and v projections of one new token per row (rows <= 16) over the concatenated weight, with RoPE(K) and
    the append to `cache` (a PagedKVCache) in the same launch; returns q (rows, num_heads * D).  Leaves in the cache
    the bits of `gemm_bf16_nt_skinny` + `cache.append`."""
    _need(x, torch.bfloat16, "gemm_qkv_append_bf16_skinny(x)")
    _need(wqkv_t, torch.bfloat16, "gemm_qkv_append_bf16_skinny(wqkv_t)")
    _need(seq_ids, torch.int32, "gemm_qkv_append_bf16_skinny(seq_ids)")
    _need(positions, torch.int32, "gemm_qkv_append_bf16_skinny(positions)")
    M, K = x.shape
    D, Hkv = cache.head_dim, cache.num_kv_heads
    if wqkv_t.shape != ((num_heads + 2 * Hkv) * D, K):
        raise RuntimeError(f"MatMul: inner dimensions mismatch {tuple(x.shape)} x {tuple(wqkv_t.shape)}^T")
    q = torch.empty((M, num_heads * D), dtype=torch.bfloat16, device=x.device)
    _lib.check(_lib.load().bn_gemm_qkv_append_bf16_skinny(
        x.data_ptr(), wqkv_t.data_ptr(), M, K, num_heads, Hkv, D, q.data_ptr(), cache.pool.data_ptr(), cache.num_pages,
        cache.page_table.data_ptr(), cache.max_pages, seq_ids.data_ptr(), positions.data_ptr(), float(cache.theta),
        _stream()))
    return q


def gemm_swiglu_bf16_nt_skinny(x: torch.Tensor, gate_t: torch.Tensor, up_t: torch.Tensor) -> torch.Tensor:
    """silu(x @ Wgate) * (x @ Wup) for at most 16 rows, the two weights (inter, K) given separately."""
    for t, n in ((x, "x"), (gate_t, "gate_t"), (up_t, "up_t")):
        _need(t, torch.bfloat16, f"gemm_swiglu_bf16_nt_skinny({n})")
    M, K = x.shape
    inter = gate_t.shape[0]
    if gate_t.shape != (inter, K) or up_t.shape != gate_t.shape:
        raise RuntimeError("gemm_swiglu_bf16_nt_skinny: gate and up weights must both be (inter, K)")
    out = torch.empty((M, inter), dtype=torch.bfloat16, device=x.device)
    _lib.check(_lib.load().bn_gemm_swiglu_bf16_nt_skinny(x.data_ptr(), gate_t.data_ptr(), up_t.data_ptr(), out.data_ptr(),
                                                         M, inter, K, _stream()))
    return out


def linear_bf16(x: torch.Tensor, weight_t: torch.Tensor) -> torch.Tensor:
    """x (rows, in) @ weight_t (out, in)^T, choosing the kernel by shape: at most 16 rows -> the weight-streaming
    kernel; few rows and too few 256-wide output tiles to occupy the GPU (measured cross-over: fewer than half as many
    tiles as SMs) -> the split-K small-M form; otherwise the large-tile kernel."""
    rows, n_out = x.shape[0], weight_t.shape[0]
    if skinny_ok(rows, n_out, x.shape[1]):
        return gemm_bf16_nt_skinny(x, weight_t)
    if rows <= 128 and (n_out + 255) // 256 < 74:
        return gemm_bf16_nt_small_m(x, weight_t)
    return gemm_bf16_nt(x, weight_t)


def add_rmsnorm_bf16(a: torch.Tensor, b: Optional[torch.Tensor], weight: torch.Tensor, eps: float = 1e-6, *,
                     want_sum: bool = True) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
    """(a + b rounded to bf16, rmsnorm of that sum) for a bf16 residual stream (tokens, hidden); b None: plain norm."""
    _need(a, torch.bfloat16, "add_rmsnorm_bf16(a)")
    _need(weight, torch.bfloat16, "add_rmsnorm_bf16(weight)")
    if b is not None:
        _need(b, torch.bfloat16, "add_rmsnorm_bf16(b)")
        if b.shape != a.shape:
            raise RuntimeError("RMSNorm: input/output shape mismatch")
    rows, hidden = a.shape
    if weight.numel() != hidden:
        raise RuntimeError("RMSNorm: weight shape must be (1, hidden_dim)")
    total = torch.empty_like(a) if (want_sum and b is not None) else None
    y = torch.empty_like(a)
    _lib.check(_lib.load().bn_add_rmsnorm_bf16(a.data_ptr(), b.data_ptr() if b is not None else None, weight.data_ptr(),
                                               total.data_ptr() if total is not None else None, y.data_ptr(), rows,
                                               hidden, float(eps), _stream()))
    return (total if b is not None else a), y


def pack_gate_up(gate_t: torch.Tensor, up_t: torch.Tensor) -> torch.Tensor:
    """Packs Wgate^T and Wup^T, each (inter, K) bf16, into the weight layout of `gemm_swiglu_bf16_nt`: for every
    block of 128 intermediate indices the 128 gate rows, then the 128 up rows (zero rows beyond inter)."""
    _need(gate_t, torch.bfloat16, "pack_gate_up(gate_t)")
    _need(up_t, torch.bfloat16, "pack_gate_up(up_t)")
    if gate_t.shape != up_t.shape or gate_t.dim() != 2:
        raise RuntimeError("pack_gate_up: gate and up weights must have the same (inter, K) shape")
    inter, K = gate_t.shape
    blocks = (inter + 127) // 128
    packed = torch.zeros((blocks, 2, 128, K), dtype=torch.bfloat16, device=gate_t.device)
    padded = torch.zeros((2, blocks * 128, K), dtype=torch.bfloat16, device=gate_t.device)
    padded[0, :inter], padded[1, :inter] = gate_t, up_t
    packed[:, 0], packed[:, 1] = padded[0].view(blocks, 128, K), padded[1].view(blocks, 128, K)
    return packed.view(blocks * 256, K)


def gemm_swiglu_bf16_nt(x: torch.Tensor, gate_up_t: torch.Tensor, inter: int, *, out: Optional[torch.Tensor] = None,
                        error_word: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(x @ Wgate) * (x @ Wup) -> (M, inter) bf16 in one launch; gate_up_t from `pack_gate_up`."""
    _need(x, torch.bfloat16, "gemm_swiglu_bf16_nt(x)")
    _need(gate_up_t, torch.bfloat16, "gemm_swiglu_bf16_nt(gate_up_t)")
    M, K = x.shape
    if gate_up_t.shape != ((inter + 127) // 128 * 256, K):
        raise RuntimeError("gemm_swiglu_bf16_nt: packed weight has the wrong shape for this inter / K")
    if out is None:
        out = torch.empty((M, inter), dtype=torch.bfloat16, device=x.device)
    _need(out, torch.bfloat16, "gemm_swiglu_bf16_nt(out)")
    _lib.check(_lib.load().bn_gemm_swiglu_bf16_nt(x.data_ptr(), gate_up_t.data_ptr(), out.data_ptr(), M, int(inter), K,
                                                  _gemm_error_ptr(x.device, error_word), _stream()))
    return out


class HostPrefillPipeline:
    """Prefill attention for callers whose q/k/v/out live in (pinned) HOST memory, as the reference's tensors do
    before `to_device()` (mygrad tensors are created on the host and copied per call).  Every `submit` copies that
    call's inputs host->device, runs the two kernels and copies the result device->host, but on three streams with
    `depth` rotating device buffers, so the copies of neighbouring calls overlap each other (PCIe is full duplex)
    and the kernels.  `finish()` makes the current stream wait for everything submitted.

    The result of submit number i is complete in its `out_host` once `finish()` (or a later synchronize) returns."""

    def __init__(self, B: int, S: int, Hq: int, Hkv: int, D: int = 64, *, depth: int = 2, device=None):
        dev = device or "cuda"
        self.shape = (B, S, Hq, Hkv, D)
        self.slots = []
        for _ in range(depth):
            self.slots.append(dict(
                q=torch.empty((B, S, Hq, D), dtype=torch.bfloat16, device=dev),
                k=torch.empty((B, S, Hkv, D), dtype=torch.bfloat16, device=dev),
                v=torch.empty((B, S, Hkv, D), dtype=torch.bfloat16, device=dev),
                o=torch.empty((B, S, Hq, D), dtype=torch.bfloat16, device=dev),
                ws=prefill_workspace(B, S, Hq, Hkv, D, dev),
                in_done=torch.cuda.Event(), run_done=torch.cuda.Event(), out_done=torch.cuda.Event(), used=False))
        self.s_in, self.s_run, self.s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        self.n = 0
        self._started = False

    def submit(self, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor, out_host: torch.Tensor, **kw):
        for t, n in ((q_host, "q"), (k_host, "k"), (v_host, "v"), (out_host, "out")):
            if t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
                raise RuntimeError(f"HostPrefillPipeline({n}): expected a contiguous bf16 host tensor")
        if not self._started:
            # work already queued on the caller's stream comes first
            ev = torch.cuda.Event()
            ev.record()
            for st in (self.s_in, self.s_run, self.s_out):
                st.wait_event(ev)
            self._started = True
        sl = self.slots[self.n % len(self.slots)]
        self.n += 1
        with torch.cuda.stream(self.s_in):
            if sl["used"]:
                self.s_in.wait_event(sl["run_done"])       # the slot's inputs are still being read until then
            sl["q"].copy_(q_host, non_blocking=True)
            sl["k"].copy_(k_host, non_blocking=True)
            sl["v"].copy_(v_host, non_blocking=True)
            sl["in_done"].record()
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(sl["in_done"])
            if sl["used"]:
                self.s_run.wait_event(sl["out_done"])      # the slot's previous result must have left the device
            attn_prefill_bf16(sl["q"], sl["k"], sl["v"], out=sl["o"], workspace=sl["ws"], **kw)
            sl["run_done"].record()
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(sl["run_done"])
            out_host.copy_(sl["o"], non_blocking=True)
            sl["out_done"].record()
        sl["used"] = True

    def finish(self) -> None:
        """The current stream waits for every submitted call (inputs copied, kernels run, results on the host)."""
        cur = torch.cuda.current_stream()
        for sl in self.slots:
            if sl["used"]:
                cur.wait_event(sl["out_done"])
        self._started = False

    def status(self) -> None:
        for sl in self.slots:
            sl["ws"].status()


def lse_combine(outs: torch.Tensor, lses: torch.Tensor, *, out_dtype=torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """outs (P, n, D) fp32, lses (P, n) fp32 -> merged (n, D), lse (n)."""
    _need(outs, torch.float32, "lse_combine(outs)")
    _need(lses, torch.float32, "lse_combine(lses)")
    P, n, D = outs.shape
    o32 = torch.empty((n, D), dtype=torch.float32, device=outs.device) if out_dtype == torch.float32 else None
    o16 = torch.empty((n, D), dtype=torch.bfloat16, device=outs.device) if out_dtype == torch.bfloat16 else None
    lse = torch.empty((n,), dtype=torch.float32, device=outs.device)
    _lib.check(_lib.load().bn_attn_lse_combine(outs.data_ptr(), lses.data_ptr(), P, n, D,
                                               o32.data_ptr() if o32 is not None else None,
                                               o16.data_ptr() if o16 is not None else None, lse.data_ptr(), _stream()))
    return (o32 if o32 is not None else o16), lse

"""Paged bf16 KV cache and single-token decode.

The reference has no cache: `generate()` recomputes the whole sequence for
every new token and keeps the last row (mygrad/llama/llama_model.py:136-144).
`PagedKVCache` supplies what that loop lacks — K (stored rotated) and V of the
earlier tokens — so that decoding one token reads each cached byte once.

Layout of the pool (one per layer):
    pool[page][kv_head][0 = K, 1 = V][16 tokens][head_dim]   bf16
`page_table[seq][logical_page]` names the pool page; pages of a sequence need
not be contiguous.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .ops import Workspace, _need, _stream

PAGE_TOKENS = _lib.BN_PAGE_TOKENS


class PagedKVCache:
    def __init__(self, num_pages: int, num_seqs: int, max_pages_per_seq: int, num_kv_heads: int = 4,
                 head_dim: int = 64, theta: float = 10000.0, device="cuda"):
        self.num_pages, self.num_seqs, self.max_pages = int(num_pages), int(num_seqs), int(max_pages_per_seq)
        self.num_kv_heads, self.head_dim, self.theta = int(num_kv_heads), int(head_dim), float(theta)
        self.pool = torch.zeros((num_pages, num_kv_heads, 2, PAGE_TOKENS, head_dim), dtype=torch.bfloat16, device=device)
        self.page_table = torch.zeros((num_seqs, max_pages_per_seq), dtype=torch.int32, device=device)
        self.seq_lens = torch.zeros((num_seqs,), dtype=torch.int32, device=device)
        self._ws = {}          # decode scratch per (B, Hq, max_seq_len, chunk_tokens); kept while the cache lives

    @property
    def max_seq_len(self) -> int:
        return self.max_pages * PAGE_TOKENS

    def append(self, seq_ids: torch.Tensor, positions: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor) -> None:
        """Writes tokens (sequence seq_ids[t], position positions[t]) with
        RoPE(K) fused; k_new, v_new (T, Hkv*D) fp32 or bf16.  Does not touch
        seq_lens (the caller advances them)."""
        T = k_new.shape[0]
        if k_new.dtype not in (torch.float32, torch.bfloat16) or v_new.dtype != k_new.dtype:
            raise RuntimeError("kv append: k/v must both be fp32 or both bf16")
        for t in (k_new, v_new):
            if not t.is_cuda:
                raise RuntimeError("kv append: only GPU implementation available")
            if t.stride(1) != 1 or t.stride(0) != k_new.stride(0):
                raise RuntimeError("kv append: k/v rows must be contiguous with equal row stride")
        _need(seq_ids, torch.int32, "kv append(seq_ids)")
        _need(positions, torch.int32, "kv append(positions)")
        _lib.check(_lib.load().bn_kv_append(
            self.pool.data_ptr(), self.num_pages, self.page_table.data_ptr(), self.max_pages, seq_ids.data_ptr(),
            positions.data_ptr(), T, k_new.data_ptr(), v_new.data_ptr(), k_new.stride(0),
            0 if k_new.dtype == torch.float32 else 1, self.num_kv_heads, self.head_dim, self.theta, _stream()))

    def workspace(self, B: int, Hq: int, max_seq_len: int, chunk_tokens: int = 0) -> Workspace:
        """The decode scratch for this shape.  A buffer, once handed out, is never freed or replaced while the
        cache lives: a captured CUDA graph may hold its address."""
        key = (B, Hq, max_seq_len, chunk_tokens)
        ws = self._ws.get(key)
        if ws is None:
            n = _lib.load().bn_attn_decode_workspace_bytes(B, Hq, self.num_kv_heads, self.head_dim, max_seq_len,
                                                          chunk_tokens)
            if n == 0:
                raise RuntimeError("bn_attn_decode_paged: unsupported shape")
            ws = self._ws[key] = Workspace(n, self.pool.device)
        return ws

    def status(self) -> None:
        """Raises if a decode launch on any of this cache's scratch buffers gave up on a bounded wait."""
        for ws in self._ws.values():
            ws.status()

    def decode(self, q: torch.Tensor, *, num_heads: int, scale: Optional[float] = None, rope_q: bool = True,
               q_positions: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
               out_f32: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None,
               max_seq_len: Optional[int] = None, chunk_tokens: int = 0, seq_lens: Optional[torch.Tensor] = None,
               page_table: Optional[torch.Tensor] = None) -> torch.Tensor:
        """q (B, Hq, D) bf16 (pre-RoPE when rope_q) -> out (B, Hq, D) bf16."""
        _need(q, torch.bfloat16, "decode(q)")
        B, Hq, D = q.shape
        seq_lens = self.seq_lens if seq_lens is None else seq_lens
        page_table = self.page_table if page_table is None else page_table
        if out is None and out_f32 is None:
            out = torch.empty_like(q)
        if max_seq_len is None:
            max_seq_len = self.max_seq_len
        if scale is None:
            scale = 1.0 / (D ** 0.5)
        ws = self.workspace(B, Hq, max_seq_len, chunk_tokens)
        _lib.check(_lib.load().bn_attn_decode_paged(
            q.data_ptr(), self.pool.data_ptr(), self.num_pages, page_table.data_ptr(), page_table.shape[1],
            seq_lens.data_ptr(), q_positions.data_ptr() if q_positions is not None else None,
            out.data_ptr() if out is not None else None, out_f32.data_ptr() if out_f32 is not None else None,
            lse.data_ptr() if lse is not None else None, B, Hq, self.num_kv_heads, D, float(scale), self.theta,
            int(bool(rope_q)), int(max_seq_len), int(chunk_tokens), ws.ptr, ws.nbytes, _stream()))
        return out if out is not None else out_f32

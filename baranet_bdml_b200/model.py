"""LLaMAModel on the bf16 path with a paged KV cache: `generate()` without whole-sequence recomputation.

Mirror of mygrad/llama/llama_model.py (`LLaMAModel`: embed_tokens, layers, norm, lm_head; `__call__`, `generate`),
composed from the rows of this package: device-side embedding gather, `LLaMADecoderLayerBF16` blocks for the prompt,
and for every new token one row per sequence through the same weights with `bn_kv_append` + `bn_attn_decode_paged`
instead of attention over the recomputed sequence (the reference recomputes the whole sequence for every token and
keeps the last row, llama_model.py:136-144), then the final norm, the lm_head GEMM and a device-side argmax.
Greedy decoding only (temperature / top-k sampling of the reference is host code).  Inference only.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from . import _lib, ops
from .kv_cache import PAGE_TOKENS, PagedKVCache
from .layers import LLaMAConfig, LLaMADecoderLayerBF16


class LLaMAModelBF16:
    def __init__(self, config: LLaMAConfig, is_cuda: bool = True):
        if not is_cuda:
            raise RuntimeError("LLaMAModelBF16: only GPU implementation available")
        self.config = config
        # embed_tokens as the reference initialises it (llama_model.py:44-50: normal, std 0.02), fp32 table
        self.embed_tokens = torch.from_numpy(
            (np.random.randn(config.vocab_size, config.hidden_size) * 0.02).astype(np.float32)).cuda()
        self.layers = [LLaMADecoderLayerBF16(config) for _ in range(config.num_hidden_layers)]
        self.norm_weight = torch.ones(config.hidden_size, dtype=torch.bfloat16, device="cuda")
        from .layers import _init_weight_t
        self.lm_head = _init_weight_t(config.hidden_size, config.vocab_size)                    # (vocab, hidden)
        self.caches: Optional[List[PagedKVCache]] = None

    # ------------------------------------------------------------------ pieces
    def embed(self, input_ids: torch.Tensor, check: bool = True) -> torch.Tensor:
        """(n,) int32 token ids on the device -> (n, hidden) bf16 (gather on the device).  `check=False` skips the
        host read of the out-of-range flag (a synchronisation), for use inside a CUDA graph."""
        ids = input_ids.to(torch.int32).contiguous()
        n, H = ids.numel(), self.config.hidden_size
        out = torch.empty((n, H), dtype=torch.float32, device="cuda")
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        _lib.check(_lib.load().bn_embedding_gather_f32(self.embed_tokens.data_ptr(), H, ids.data_ptr(), out.data_ptr(), H,
                                                       n, H, self.config.vocab_size, err.data_ptr(),
                                                       torch.cuda.current_stream().cuda_stream))
        if check and int(err.item()) != 0:
            raise IndexError("token id out of range")
        return out.to(torch.bfloat16)

    def _logits(self, residual: torch.Tensor, pending: torch.Tensor) -> torch.Tensor:
        """final norm of (residual + pending), lm_head: (rows, hidden) -> (rows, vocab) fp32"""
        _, normed = ops.add_rmsnorm_bf16(residual, pending, self.norm_weight, self.config.rms_norm_eps, want_sum=False)
        return ops.gemm_bf16_nt(normed, self.lm_head).float()

    def argmax(self, logits: torch.Tensor) -> torch.Tensor:
        rows, cols = logits.shape
        out = torch.zeros((rows,), dtype=torch.int32, device="cuda")
        _lib.check(_lib.load().bn_argmax_rows_f32(logits.data_ptr(), logits.stride(0), logits.stride(1), out.data_ptr(),
                                                  rows, cols, torch.cuda.current_stream().cuda_stream))
        return out

    # ----------------------------------------------------------------- forward
    def __call__(self, input_ids: torch.Tensor, position_offset: int = 0, use_causal_mask: bool = True) -> torch.Tensor:
        """Whole-sequence forward as the reference's `__call__` (llama_model.py:80-110): (B, S) ids -> (B, S, vocab)."""
        B, S = input_ids.shape
        h = self.embed(input_ids.reshape(-1)).view(B, S, -1)
        pending = None
        for layer in self.layers:
            h, pending = layer.forward_parts(h, position_offset, use_causal_mask, pending=pending)
        H = self.config.hidden_size
        return self._logits(h.reshape(B * S, H), pending.reshape(B * S, H)).view(B, S, -1)

    def _alloc_caches(self, B: int, max_len: int):
        cfg = self.config
        pages_per_seq = (max_len + PAGE_TOKENS - 1) // PAGE_TOKENS
        self.caches = []
        for _ in self.layers:
            c = PagedKVCache(B * pages_per_seq, B, pages_per_seq, cfg.num_key_value_heads, cfg.head_dim, cfg.rope_theta)
            c.page_table.copy_(torch.arange(B * pages_per_seq, dtype=torch.int32, device="cuda").view(B, pages_per_seq))
            if self.caches:
                c.seq_lens = self.caches[0].seq_lens      # every block holds the same tokens: ONE length vector, advanced once per step
            self.caches.append(c)
        self.seq_lens = self.caches[0].seq_lens

    def prefill(self, input_ids: torch.Tensor, max_len: int) -> torch.Tensor:
        """Prompt pass: (B, S) ids -> logits of the last position (B, vocab); fills the KV caches."""
        cfg = self.config
        B, S = input_ids.shape
        self._alloc_caches(B, max_len)
        h = self.embed(input_ids.reshape(-1)).view(B, S, -1)
        pending = None
        H = cfg.hidden_size
        # one scratch buffer for all blocks (they run one after the other): cos/sin table written once
        ws = ops.prefill_workspace(B, S, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim)
        ops.prefill_table(ws, B, S, cfg.num_key_value_heads, cfg.head_dim, cfg.rope_theta, 0)
        for layer, cache in zip(self.layers, self.caches):
            x2 = h.reshape(B * S, H)
            residual, normed = ops.add_rmsnorm_bf16(x2, None if pending is None else pending.reshape(B * S, H),
                                                    layer.input_layernorm_weight, layer.eps)
            at = layer.self_attn
            # q/k/v in one GEMM whose epilogue rotates K and appends K and V to this block's cache
            attn = at.attend(normed, B, S, 0, True, cache=cache, workspace=ws)
            o = ops.gemm_bf16_nt(attn, at.o_proj)
            residual, normed = ops.add_rmsnorm_bf16(residual, o, layer.post_attention_layernorm_weight, layer.eps)
            h, pending = residual.view(B, S, H), layer.mlp(normed).view(B, S, H)
        self.seq_lens.fill_(S)
        return self._logits(h[:, -1].contiguous(), pending[:, -1].contiguous())

    def decode_step(self, token_ids: torch.Tensor, check: bool = True) -> torch.Tensor:
        """One new token per sequence: (B,) ids -> (B, vocab) logits; appends to the caches."""
        B = token_ids.numel()
        h = self.embed(token_ids, check)
        seq_ids = torch.arange(B, dtype=torch.int32, device="cuda")
        pending = None
        positions = self.seq_lens.clone()                         # the new token's position = current length
        self.seq_lens.add_(1)
        for layer, cache in zip(self.layers, self.caches):
            residual, normed = ops.add_rmsnorm_bf16(h, pending, layer.input_layernorm_weight, layer.eps)
            at = layer.self_attn
            kv = at.num_kv_heads * at.head_dim
            if ops.skinny_ok(B, at.hidden_size + 2 * kv, normed.shape[1]):
                # q, k, v as one stream of the concatenated weight; K rotated and K, V appended by the same launch
                q = ops.gemm_qkv_append_bf16_skinny(normed, at.packed_qkv(), cache, seq_ids, positions, at.num_heads)
                q = q.view(B, at.num_heads, at.head_dim)
            else:
                q = ops.linear_bf16(normed, at.q_proj).view(B, at.num_heads, at.head_dim)
                k = ops.linear_bf16(normed, at.k_proj)
                v = ops.linear_bf16(normed, at.v_proj)
                cache.append(seq_ids, positions, k, v)
            attn = cache.decode(q, num_heads=at.num_heads, scale=float(at.scale))      # RoPE(q) at position len - 1
            o = ops.linear_bf16(attn.view(B, -1), at.o_proj)
            residual, normed = ops.add_rmsnorm_bf16(residual, o, layer.post_attention_layernorm_weight, layer.eps)
            h, pending = residual, layer.mlp(normed, few_rows=True)
        return self._logits(h, pending)

    def capture_decode_step(self):
        """Captures `decode_step` + argmax for the current batch into a CUDA graph: a step is about 30 launches that
        Python issues one by one (the host, not the GPU, bounds it); replayed from a graph they are one submission.
        Returns step(token_ids) -> (logits, next_ids), both static buffers overwritten by the next call.  The caches'
        lengths advance inside the graph, so every replay is the next position."""
        B = self.caches[0].num_seqs
        static_tok = torch.zeros((B,), dtype=torch.int32, device="cuda")
        saved = self.seq_lens.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                      # warm-up outside the capture (workspaces, attributes)
            self.decode_step(static_tok, check=False)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            logits = self.decode_step(static_tok, check=False)
            nxt = self.argmax(logits)
        torch.cuda.synchronize()
        self.seq_lens.copy_(saved)                         # warm-up and capture must not count as positions

        def step(token_ids: torch.Tensor):
            static_tok.copy_(token_ids)
            graph.replay()
            return logits, nxt

        step.graph = graph
        return step

    def generate(self, input_ids: np.ndarray, max_new_tokens: int = 50) -> List[List[int]]:
        """Greedy `generate` (llama_model.py:112-168 with temperature -> 0): prompts (B, S) of equal length."""
        ids = torch.from_numpy(np.ascontiguousarray(input_ids, dtype=np.int32)).cuda()
        if ids.dim() == 1:
            ids = ids[None]
        B, S = ids.shape
        logits = self.prefill(ids, S + max_new_tokens)
        out = [list(map(int, row)) for row in ids.cpu().numpy()]
        done = [False] * B
        for _ in range(max_new_tokens):
            nxt = self.argmax(logits)
            host = nxt.cpu().numpy()
            for b in range(B):
                if not done[b]:
                    if int(host[b]) == self.config.eos_token_id:
                        done[b] = True
                    else:
                        out[b].append(int(host[b]))
            if all(done):
                break
            logits = self.decode_step(nxt)
        return out

    def status(self) -> None:
        """Raises if any kernel of the model gave up a bounded wait since the last check (attention scratch of every
        block's cache, and the per-device error word of the projection GEMMs).  Synchronises."""
        for c in self.caches or []:
            c.status()
        ops.gemm_status()

    def parameters(self):
        p = [self.embed_tokens]
        for layer in self.layers:
            p.extend(layer.parameters())
        return p + [self.norm_weight, self.lm_head]

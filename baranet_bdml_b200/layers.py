"""Drop-in mirror of the reference's attention layer.

`GroupedQueryAttention` keeps the constructor, attributes, call signature and
`parameters()` of mygrad/llama/llama_layers.py:46-191; only the body between
the projections changes: the steps rope -> repeat_kv -> q k^T -> *scale ->
softmax -> p v (llama_layers.py:161-183: four host round trips, seven launches
and an (S,S) matrix in memory) become ONE fused call.

Two semantics are offered (see `heads_mode`):
  "collapsed"  exactly what the reference computes: its `_split_heads` is a
               no-op (llama_layers.py:87-103), so there is ONE softmax over the
               scores summed over all heads.  Default, because it is what makes
               the layer a numerical drop-in.
  "per_head"   standard grouped-query attention, one softmax per query head.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import _lib
from .tensor import AGTensor, TensorF

try:  # only for annotations
    import torch  # noqa: F401
except Exception:  # pragma: no cover
    torch = None


@dataclass
class LLaMAConfig:
    """Field-for-field mirror of mygrad/llama/llama_config.py:8-38."""
    vocab_size: int = 32000
    hidden_size: int = 2048
    intermediate_size: int = 5632
    num_hidden_layers: int = 22
    num_attention_heads: int = 32
    num_key_value_heads: int = 4
    max_position_embeddings: int = 2048
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    pad_token_id: int = 0
    bos_token_id: int = 1
    eos_token_id: int = 2

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def num_key_value_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def __post_init__(self):
        assert self.hidden_size % self.num_attention_heads == 0
        assert self.num_attention_heads % self.num_key_value_heads == 0


class RMSNorm:
    """mygrad/llama/llama_layers.py:13-29: same constructor, `weight` (1, hidden) initialised to ones, `__call__`,
    `parameters()`.  `add_norm(residual, x)` is the fused form of the decoder layer's residual add followed by this
    norm (llama_layers.py:279-283): returns (residual + x, norm(residual + x)) from one launch."""

    def __init__(self, hidden_size: int, eps: float = 1e-6, is_cuda: bool = True):
        self.hidden_size = hidden_size
        self.eps = eps
        self.is_cuda = is_cuda
        self.weight = AGTensor(np.ones((1, hidden_size), dtype=np.float32), requires_grad=True, is_cuda=is_cuda)

    def __call__(self, x: AGTensor) -> AGTensor:
        return x.rmsnorm(self.weight, self.eps)

    def add_norm(self, residual: AGTensor, x: AGTensor):
        return residual.add_rmsnorm(x, self.weight, self.eps)

    def parameters(self):
        return [self.weight]


class RotaryEmbedding:
    """mygrad/llama/llama_layers.py:32-42."""

    def __init__(self, dim: int, max_position_embeddings: int = 2048, base: float = 10000.0):
        self.dim = dim
        self.max_position_embeddings = max_position_embeddings
        self.base = base

    def __call__(self, x: AGTensor, position_offset: int = 0) -> AGTensor:
        return x.rope(position_offset=position_offset, head_dim=self.dim, theta=self.base)


class GroupedQueryAttention:
    """mygrad/llama/llama_layers.py:46-191 with the attention core fused."""

    def __init__(self, config, is_cuda: bool = True, heads_mode: str = "collapsed"):
        if heads_mode not in ("collapsed", "per_head"):
            raise ValueError("heads_mode must be 'collapsed' or 'per_head'")
        self.config = config
        self.is_cuda = is_cuda
        self.heads_mode = heads_mode
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = config.num_key_value_heads
        self.head_dim = config.head_dim
        self.hidden_size = config.hidden_size
        self.q_proj = self._init_linear(self.hidden_size, self.hidden_size)
        self.k_proj = self._init_linear(self.hidden_size, self.num_kv_heads * self.head_dim)
        self.v_proj = self._init_linear(self.hidden_size, self.num_kv_heads * self.head_dim)
        self.o_proj = self._init_linear(self.hidden_size, self.hidden_size)
        self.rotary_emb = RotaryEmbedding(self.head_dim, max_position_embeddings=config.max_position_embeddings,
                                          base=config.rope_theta)
        self.scale = 1.0 / np.sqrt(self.head_dim)

    def _init_linear(self, in_features: int, out_features: int) -> AGTensor:
        # Xavier/Glorot, as llama_layers.py:80-85
        std = np.sqrt(2.0 / (in_features + out_features))
        w = np.random.randn(in_features, out_features).astype(np.float32) * std
        return AGTensor(w, requires_grad=True, is_cuda=self.is_cuda)

    def __call__(self, hidden_states: AGTensor, position_offset: int = 0, use_causal_mask: bool = True) -> AGTensor:
        query = hidden_states @ self.q_proj
        key = hidden_states @ self.k_proj
        value = hidden_states @ self.v_proj
        mode = _lib.BN_HEADS_COLLAPSED if self.heads_mode == "collapsed" else _lib.BN_HEADS_PER_HEAD
        attn = query.data.attention_fused(
            key.data, value.data, float(self.scale), causal=use_causal_mask, seq_offset=position_offset,
            num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
            theta=self.rotary_emb.base, heads_mode=mode)
        attn_output = AGTensor(attn, (query, key, value), "attention_fused", requires_grad=False)
        return attn_output @ self.o_proj

    def parameters(self):
        return [self.q_proj, self.k_proj, self.v_proj, self.o_proj]


_DEVICE_INIT = None     # (std, torch.Generator) while `device_init` is active


class device_init:
    """Within this context the bf16 layers draw their weights on the GPU from N(0, std) instead of the reference's
    Xavier initialisation on the host (mygrad/llama/llama_layers.py:80-85): for benchmarks at full model size,
    where a billion host-side normal draws would take longer than the measurement."""

    def __init__(self, std: float, seed: int = 0):
        self.std, self.seed = float(std), int(seed)

    def __enter__(self):
        import torch
        global _DEVICE_INIT
        _DEVICE_INIT = (self.std, torch.Generator(device="cuda").manual_seed(self.seed))
        return self

    def __exit__(self, *exc):
        global _DEVICE_INIT
        _DEVICE_INIT = None
        return False


def _init_weight_t(in_features: int, out_features: int):
    """(out_features, in_features) bf16 on the GPU: the weight of `x @ W` held transposed."""
    import torch
    if _DEVICE_INIT is not None:
        std, gen = _DEVICE_INIT
        return (torch.randn((out_features, in_features), generator=gen, device="cuda") * std).to(torch.bfloat16)
    std = np.sqrt(2.0 / (in_features + out_features))          # Xavier/Glorot as llama_layers.py:80-85
    w = np.random.randn(in_features, out_features).astype(np.float32) * std
    return torch.from_numpy(np.ascontiguousarray(w.T)).cuda().to(torch.bfloat16)


class GroupedQueryAttentionBF16:
    """The same layer on the bf16 tensor-core path, per-head grouped-query attention (BASELINE configs 2-4): q, k and
    v come from ONE tensor-core GEMM (`bn_gemm_qkv_rope_bf16`: weights held transposed, (out_features, in_features),
    bf16; RoPE(K) in its epilogue), the core is `bn_attn_prefill_bf16` (RoPE(Q), causal softmax, P V fused), o_proj
    is `bn_gemm_bf16_nt`: three kernel launches.  Same constructor arguments, attribute names and
    `__call__(hidden_states, position_offset, use_causal_mask)` as mygrad/llama/llama_layers.py:46-191;
    hidden_states is a torch bf16 tensor (B, S, hidden) or (S, hidden) on the GPU.  Inference only."""

    def __init__(self, config, is_cuda: bool = True):
        import torch
        if not is_cuda:
            raise RuntimeError("Attention: only GPU implementation available")
        self.config = config
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = config.num_key_value_heads
        self.head_dim = config.head_dim
        self.hidden_size = config.hidden_size
        kv = self.num_kv_heads * self.head_dim

        init = _init_weight_t
        self.q_proj, self.k_proj = init(self.hidden_size, self.hidden_size), init(self.hidden_size, kv)
        self.v_proj, self.o_proj = init(self.hidden_size, kv), init(self.hidden_size, self.hidden_size)
        self._qkv_t = None          # Wq^T, Wk^T, Wv^T stacked: built at the first fused call from the three above
        self._ws_table = None       # (S, theta, position_offset) of the cos/sin table in the scratch buffer
        self.rotary_emb = RotaryEmbedding(self.head_dim, max_position_embeddings=config.max_position_embeddings,
                                          base=config.rope_theta)
        self.scale = 1.0 / np.sqrt(self.head_dim)
        self._ws = None

    def packed_qkv(self):
        """(Hq + 2 Hkv) * D rows: the three projection weights (held transposed) one after the other.  Rebuilt when
        one of them has been replaced (they are plain attributes, as in the reference layer)."""
        import torch
        key = (self.q_proj.data_ptr(), self.k_proj.data_ptr(), self.v_proj.data_ptr())
        if self._qkv_t is None or self._qkv_t[0] != key:
            self._qkv_t = (key, torch.cat([self.q_proj, self.k_proj, self.v_proj], dim=0).contiguous())
        return self._qkv_t[1]

    def attend(self, x2, B: int, S: int, position_offset: int = 0, use_causal_mask: bool = True, cache=None,
               workspace=None):
        """x2 (B*S, hidden) bf16 -> attention output before o_proj, (B*S, hidden): ONE GEMM for q, k, v with the K
        rotation (and, with `cache`, the append of K and V at positions position_offset ..) in its epilogue, then the
        fused attention kernel on the rotated K it left in the scratch buffer.  head_dim 64.  A caller that passes
        its own `workspace` keeps its cos/sin table current itself (ops.prefill_table)."""
        from . import ops
        if workspace is None:
            key = (B, S)
            if self._ws is None or self._ws[0] != key:
                self._ws = (key, ops.prefill_workspace(B, S, self.num_heads, self.num_kv_heads, self.head_dim, x2.device))
                self._ws_table = None
            workspace = self._ws[1]
            tkey = (S, float(self.rotary_emb.base), int(position_offset))
            if self._ws_table != tkey:
                ops.prefill_table(workspace, B, S, self.num_kv_heads, self.head_dim, self.rotary_emb.base, position_offset)
                self._ws_table = tkey
        q, v = ops.gemm_qkv_rope_bf16(x2, self.packed_qkv(), B, S, self.num_heads, self.num_kv_heads, self.head_dim,
                                      workspace, position_offset=position_offset, cache=cache)
        attn = ops.attn_prefill_bf16(q, None, v, scale=float(self.scale), theta=self.rotary_emb.base,
                                     position_offset=position_offset, causal=use_causal_mask, workspace=workspace,
                                     reuse_rotated_k=True)
        return attn.view(B * S, self.num_heads * self.head_dim)

    def __call__(self, hidden_states, position_offset: int = 0, use_causal_mask: bool = True):
        from . import ops
        x = hidden_states if hidden_states.dim() == 3 else hidden_states[None]
        B, S, H = x.shape
        if H != self.hidden_size:
            raise RuntimeError("Attention: hidden size mismatch")
        attn = self.attend(x.reshape(B * S, H), B, S, position_offset, use_causal_mask)
        out = ops.gemm_bf16_nt(attn, self.o_proj).view(B, S, H)
        return out if hidden_states.dim() == 3 else out[0]

    def parameters(self):
        return [self.q_proj, self.k_proj, self.v_proj, self.o_proj]


class MLPBF16:
    """The SwiGLU feed-forward block (mygrad/llama/llama_layers.py:194-235: gate_proj, up_proj, down_proj;
    `(SiLU(x @ gate) * (x @ up)) @ down`) on the tensor-core path: one fused gate/up GEMM with the SiLU * mul epilogue
    and one down GEMM.  Weights are held transposed in bf16; `gate_proj` / `up_proj` / `down_proj` keep the reference's
    names.  x: torch bf16 (tokens, hidden) on the GPU.  Inference only."""

    def __init__(self, config, is_cuda: bool = True):
        import torch
        from . import ops
        if not is_cuda:
            raise RuntimeError("MatMul: only GPU implementation available")
        self.config = config
        hidden, inter = config.hidden_size, config.intermediate_size

        init = _init_weight_t
        self.gate_proj, self.up_proj, self.down_proj = init(hidden, inter), init(hidden, inter), init(inter, hidden)
        self.intermediate_size = inter
        self._gate_up = ops.pack_gate_up(self.gate_proj, self.up_proj)

    def __call__(self, x, few_rows: bool = False):
        from . import ops
        if few_rows and ops.skinny_ok(x.shape[0], self.intermediate_size, x.shape[1]) and \
                ops.skinny_ok(x.shape[0], x.shape[1], self.intermediate_size):
            # a decode step with at most 16 rows: both products are weight streams
            h = ops.gemm_swiglu_bf16_nt_skinny(x, self.gate_proj, self.up_proj)
            return ops.gemm_bf16_nt_skinny(h, self.down_proj)
        h = ops.gemm_swiglu_bf16_nt(x, self._gate_up, self.intermediate_size)
        # the down projection has few output tiles: with few rows (a decode step) the split-K form streams its weight
        # with all SMs
        return ops.linear_bf16(h, self.down_proj) if few_rows else ops.gemm_bf16_nt(h, self.down_proj)

    def parameters(self):
        return [self.gate_proj, self.up_proj, self.down_proj]


class LLaMADecoderLayerBF16:
    """mygrad/llama/llama_layers.py:238-296 (pre-norm decoder block: input_layernorm -> self_attn -> residual add ->
    post_attention_layernorm -> mlp -> residual add) on the bf16 tensor-core path, 7 kernel launches per call:
    norm, fused q/k/v GEMM (K rotation in its epilogue), fused attention, o_proj GEMM, fused residual add + norm,
    fused gate/up GEMM, down GEMM; the last residual add is returned un-added together with the MLP output by `forward_parts`, so that
    the NEXT layer's fused add + norm performs it (`__call__` adds it for a stand-alone layer).
    hidden_states: torch bf16 (B, S, hidden) on the GPU.  Inference only."""

    def __init__(self, config, is_cuda: bool = True):
        import torch
        self.config = config
        self.self_attn = GroupedQueryAttentionBF16(config, is_cuda)
        self.mlp = MLPBF16(config, is_cuda)
        self.input_layernorm_weight = torch.ones(config.hidden_size, dtype=torch.bfloat16, device="cuda")
        self.post_attention_layernorm_weight = torch.ones(config.hidden_size, dtype=torch.bfloat16, device="cuda")
        self.eps = config.rms_norm_eps

    def forward_parts(self, hidden_states, position_offset: int = 0, use_causal_mask: bool = True, pending=None):
        """Returns (residual, mlp_out) with the layer output = residual + mlp_out.  `pending` is the previous layer's
        not-yet-added MLP output: it is added to hidden_states by this layer's first (fused) norm."""
        from . import ops
        B, S, H = hidden_states.shape
        x2 = hidden_states.reshape(B * S, H)
        residual, normed = ops.add_rmsnorm_bf16(x2, None if pending is None else pending.reshape(B * S, H),
                                                self.input_layernorm_weight, self.eps)
        attn = self.self_attn(normed.view(B, S, H), position_offset, use_causal_mask).reshape(B * S, H)
        residual, normed = ops.add_rmsnorm_bf16(residual, attn, self.post_attention_layernorm_weight, self.eps)
        return residual.view(B, S, H), self.mlp(normed).view(B, S, H)

    def __call__(self, hidden_states, position_offset: int = 0, use_causal_mask: bool = True):
        residual, mlp_out = self.forward_parts(hidden_states, position_offset, use_causal_mask)
        return residual + mlp_out

    def parameters(self):
        return ([self.input_layernorm_weight] + self.self_attn.parameters() + [self.post_attention_layernorm_weight] +
                self.mlp.parameters())


class GraphedDecoderLayerBF16:
    """`LLaMADecoderLayerBF16.forward_parts` for one fixed input shape, captured once into a CUDA graph and replayed:
    the ten launches of a block go to the GPU as one submission, without the host-side work between them (tensor-map
    encoding, argument checks, allocator calls).  `__call__(x)` copies x into the graph's static input and returns
    the static outputs (residual, mlp_out); they are overwritten by the next call."""

    def __init__(self, layer: "LLaMADecoderLayerBF16", example: "torch.Tensor", position_offset: int = 0,
                 use_causal_mask: bool = True):
        import torch
        self.layer = layer
        self.static_in = example.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):              # warm-up outside the capture: attributes, workspaces, caches
            for _ in range(2):
                layer.forward_parts(self.static_in, position_offset, use_causal_mask)
        torch.cuda.current_stream().wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_out = layer.forward_parts(self.static_in, position_offset, use_causal_mask)

    def __call__(self, hidden_states):
        self.static_in.copy_(hidden_states)
        self.graph.replay()
        return self.static_out

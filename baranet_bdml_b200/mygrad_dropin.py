"""Switches the reference's own attention layer to the fused kernel, with no change to its model code.

`install(layers_module)` rebinds `GroupedQueryAttention.__call__` of the reference's
`mygrad.llama.llama_layers` (mygrad/llama/llama_layers.py:140-188).  The projections stay the reference's
`AGTensor @ AGTensor` (op_mm); the lines from `query = self.rotary_emb(query, ...)` to
`attn_output = attn_probs @ value` (:161-183: two RoPE launches, two host round trips in `_repeat_kv`, Q K^T,
the scale, the causal softmax and P V) become ONE call of `TensorF.attention_fused`, the entry that the superset
`bten` module (baranet_bdml_b200/binding/bten_b200.cu) adds.  `uninstall` puts the original method back.

Needs a `bten` that has the entry (`bten.has_b200_attention`); with the reference's stock module `install`
raises instead of falling back.  The fused call is inference-only: its result carries no backward closure
(the reference's own gradient flow through this layer already stops at `_repeat_kv`, which creates a fresh leaf).
"""
from __future__ import annotations

_ORIGINAL = {}


def fused_call(self, hidden_states, position_offset: int = 0, use_causal_mask: bool = True):
    import sys
    AGTensor = sys.modules[type(hidden_states).__module__].AGTensor
    query = hidden_states @ self.q_proj
    key = hidden_states @ self.k_proj
    value = hidden_states @ self.v_proj
    attn = query.data.attention_fused(key.data, value.data, float(self.scale), bool(use_causal_mask),
                                      int(position_offset), num_heads=self.num_heads,
                                      num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                                      theta=float(self.rotary_emb.base))       # heads_mode 0: the reference's result
    attn_output = AGTensor(attn, (query, key, value), "attention_fused", requires_grad=False)
    return attn_output @ self.o_proj


def install(layers_module) -> None:
    """layers_module: the imported `mygrad.llama.llama_layers` of the reference tree."""
    import sys
    bten = sys.modules.get("bten")
    if bten is None or not getattr(bten, "has_b200_attention", False):
        raise RuntimeError("the loaded `bten` has no attention_fused entry: build the superset module "
                           "(make -C oracle bten REF=<reference tree>) and put it first on sys.path")
    cls = layers_module.GroupedQueryAttention
    if cls not in _ORIGINAL:
        _ORIGINAL[cls] = cls.__call__
    cls.__call__ = fused_call


def uninstall(layers_module) -> None:
    cls = layers_module.GroupedQueryAttention
    if cls in _ORIGINAL:
        cls.__call__ = _ORIGINAL.pop(cls)

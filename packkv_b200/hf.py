"""Drop-in for the attention modules of the installed transformers (5.x).

The reference ships patched copies of the model files (models/llama.py:259-282 and
models/model_adoption.md: cache created in the CausalLM forward, `past_key_value.update(...)`
followed by the eager attention).  The installed library already routes every attention module
through a registry of attention functions, so the same effect needs no model copies:

    from packkv_b200 import hf
    hf.register()                                   # once per process
    model.set_attn_implementation("packkv")
    cache = hf.make_cache(model.config, batch_size) # PackKVCacheConfigStatic.config must be set
    out = model(input_ids, past_key_values=cache, use_cache=True)      # prefill: dense K/V, eager math
    out = model(next_ids, past_key_values=cache, use_cache=True)       # decode: fused decompress-attention

Prefill (more than one query token) runs the library's eager attention on the dense K/V the
cache returns, exactly like the reference.  A decode step gets `PackKVHandle`s from the cache and
runs `PackKVCache.attend`.  All sequences of a batch advance together; padding masks are not
supported at decode (the reference's cache has the same restriction).
"""
from __future__ import annotations

from typing import Optional

import torch

from .cache import PackKVCache, PackKVHandle

ATTN_NAME = "packkv"


def packkv_attention_forward(module, query: torch.Tensor, key, value, attention_mask: Optional[torch.Tensor],
                             scaling: Optional[float] = None, dropout: float = 0.0, **kwargs):
    """Attention function with the signature of transformers' `eager_attention_forward`."""
    if isinstance(key, PackKVHandle):
        if scaling is None:
            scaling = query.shape[-1] ** -0.5
        return key.cache.attend(query, key.layer_idx, scaling), None
    from transformers.models.llama.modeling_llama import eager_attention_forward
    return eager_attention_forward(module, query, key, value, attention_mask, scaling=scaling, dropout=dropout, **kwargs)


def register(name: str = ATTN_NAME) -> str:
    """Registers the attention function (and the eager mask builder it needs) under `name`."""
    from transformers import AttentionInterface, AttentionMaskInterface
    from transformers.masking_utils import eager_mask
    AttentionInterface.register(name, packkv_attention_forward)
    AttentionMaskInterface.register(name, eager_mask)
    return name


def make_cache(config, batch_size: int, materialize: bool = False) -> PackKVCache:
    """Cache for a transformers model config: llama / mistral / qwen3 style (head_dim 128) or phi-3 style (head_dim 96,
    hidden_size // num_attention_heads)."""
    head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
    return PackKVCache(batch_size, config.num_attention_heads, head_dim, config.num_hidden_layers,
                       materialize=materialize, decode_handles=not materialize)

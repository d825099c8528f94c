"""Decode steps of a HF-transformers model served by the fused attention kernel.

The reference's caches hand dense K/V back from ``update`` and the model's own attention reads
them (``decode_impl: 'materialize_dense'``, float_cache_utils.py:1342).  This module wires the
other route: inside ``fused_decode(cache)`` a single-token ``update`` only appends (same packing
schedule, same adjuster steps) and returns the new token's K/V, and the attention function
registered here as ``'float11_fused'`` computes the step with ``adacode_decode_attn`` straight
from the packed planes.  Prefill and everything outside the context manager go through SDPA on
the dense tensors, as before.

    model.config._attn_implementation = 'float11_fused'     # after register()
    cache = Float11Cache(model.config, ...)
    with fused_decode(cache):
        out = model.generate(ids, past_key_values=cache, ...)

Limits: every cached token is attended to (no padding mask, no sliding window), head_dim 64 or
128.  Results are close to, not bit-identical with, the
materialising path (different summation order), so generated tokens can differ where two
logits are nearly tied.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch

ATTENTION_NAME = 'float11_fused'
_active_cache = None


def float11_fused_attention(module, query, key, value, attention_mask, dropout: float = 0.0,
                            scaling: Optional[float] = None, **kwargs):
    """Attention function with the ``AttentionInterface`` signature."""
    cache = _active_cache
    if cache is not None and query.shape[2] == 1 and getattr(cache, '_fused_decode', False):
        layer = cache.layers[module.layer_idx]
        out = layer.decode_attention(query, scale=scaling)           # [B, Hq, 1, D]
        return out.transpose(1, 2).contiguous(), None               # [B, 1, Hq, D]
    from transformers.integrations.sdpa_attention import sdpa_attention_forward
    return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout, scaling=scaling,
                                  **kwargs)


def register() -> str:
    """Register the attention function with transformers; returns its name."""
    from transformers import AttentionInterface
    AttentionInterface.register(ATTENTION_NAME, float11_fused_attention)
    return ATTENTION_NAME


@contextlib.contextmanager
def fused_decode(cache):
    """Single-token updates of ``cache`` skip the dense rebuild while this context is active."""
    global _active_cache
    previous = _active_cache
    _active_cache = cache
    cache._fused_decode = True
    try:
        yield cache
    finally:
        cache._fused_decode = False
        _active_cache = previous

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

Limits: every cached token is attended to, head_dim 64 or 128.  A step whose attention mask hides
any cached position (left-padded batches) or whose layer uses a sliding window cannot be served by
the kernel; such a step raises instead of attending to the wrong tokens, and ``fused_decode``
refuses a model whose attention implementation is not the one registered here (its SDPA would see
one token only).  Results are close to, not bit-identical with, the materialising path
(different summation order), so generated tokens can differ where two logits are nearly tied.
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
        if getattr(module, 'sliding_window', None):
            raise NotImplementedError('float11_fused attention has no sliding window; use the materialising path')
        if attention_mask is not None and not _mask_shows_everything(cache, attention_mask):
            raise NotImplementedError('float11_fused attention attends to every cached token, but this step\'s '
                                      'attention mask hides some (left padding?); use the materialising path')
        out = layer.decode_attention(query, scale=scaling)           # [B, Hq, 1, D]
        return out.transpose(1, 2).contiguous(), None               # [B, 1, Hq, D]
    from transformers.integrations.sdpa_attention import sdpa_attention_forward
    return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout, scaling=scaling,
                                  **kwargs)


def _mask_shows_everything(cache, mask: torch.Tensor) -> bool:
    """True when a boolean mask is all True or an additive mask is all zero.  All layers of a
    forward pass get the same mask object, so the (synchronising) check runs once per step."""
    seen = getattr(cache, '_fused_mask_seen', None)
    if seen is not None and seen[0] is mask:
        return seen[1]
    ok = bool(mask.all()) if mask.dtype == torch.bool else bool((mask == 0).all())
    cache._fused_mask_seen = (mask, ok)
    return ok


def register() -> str:
    """Register the attention function with transformers; returns its name."""
    from transformers import AttentionInterface
    AttentionInterface.register(ATTENTION_NAME, float11_fused_attention)
    return ATTENTION_NAME


@contextlib.contextmanager
def fused_decode(cache, model=None):
    """Single-token updates of ``cache`` skip the dense rebuild while this context is active.
    Pass the model (or its config) to have its attention implementation checked: with any other
    implementation the model's own attention would run on the one token ``update`` returns."""
    global _active_cache
    if model is not None:
        cfg = getattr(model, 'config', model)
        impl = getattr(cfg, '_attn_implementation', None)
        if impl != ATTENTION_NAME:
            raise RuntimeError(f"fused_decode needs config._attn_implementation == '{ATTENTION_NAME}' "
                               f'(call hf_attention.register() and set it); found {impl!r}')
    previous = _active_cache
    _active_cache = cache
    cache._fused_decode = True
    try:
        yield cache
    finally:
        cache._fused_decode = False
        cache._fused_mask_seen = None
        _active_cache = previous

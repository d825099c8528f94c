"""Calibration producer: exponent histograms of a live KV cache, in the JSON layout that
``export_initial_compress_parameters`` consumes.

Covers the part of the reference's ``export_kvcache_status.py`` that feeds the float11 cache:
``get_exp_freq_list`` for bf16 (:127-150; a Triton exponent-extraction kernel followed by
``torch.bincount``), ``extract_exp_freq`` with ``freq_type='exp'`` (:271-296) and
``merge_exp_freq`` (:298-307).  The histogram itself is one launch of ``adacode_hist_bf16`` per
tensor slice, no per-element byte buffer.  Sign / mantissa / all-bits statistics and the
fp16 / fp8 variants serve the reference's analysis scripts, not the cache path, and are not
provided.
"""
from __future__ import annotations

import torch

from . import codec


def get_exp_freq_list(t: torch.Tensor, dtype: str = 'bf16') -> list:
    """256 counts of the bf16 exponent field of ``t`` (reference: :127-150)."""
    if str(dtype).replace('torch.', '') not in ('bf16', 'bfloat16'):
        raise NotImplementedError("only dtype='bf16' feeds the float11 cache path")
    if t.numel() == 0:
        return [0] * 256
    if t.dtype != torch.bfloat16:
        t = t.to(torch.bfloat16)
    x = t.reshape(1, 1, -1, t.shape[-1]) if t.dim() != 4 else t
    if x.stride(-1) != 1:
        x = x.contiguous()
    return [int(v) for v in codec.read_back(codec.exponent_hist(x))]


def _slice_prefill_decode(tensor: torch.Tensor, prefill_len: int):
    """reference: :216-224."""
    if tensor.ndim < 2:
        raise ValueError(f'Cache tensor must have a sequence dimension, got shape={tuple(tensor.shape)}')
    seq_len = int(tensor.shape[-2])
    prefix_len = min(int(prefill_len), seq_len)
    return tensor.narrow(-2, 0, prefix_len), tensor.narrow(-2, prefix_len, seq_len - prefix_len)


def _layer_tensor_groups(kv_cache, layer_idx: int) -> dict:
    """Keys and values of one layer of a ``DynamicCache``-style object (reference: :227-268,
    ``backend='traditional_kv'``)."""
    groups = {}
    layer = kv_cache.layers[layer_idx] if hasattr(kv_cache, 'layers') else None
    if layer is not None:
        for name, attr in (('keys', 'keys'), ('values', 'values'), ('keys', 'key_cache'), ('values', 'value_cache')):
            value = getattr(layer, attr, None)
            if isinstance(value, torch.Tensor) and name not in groups:
                groups[name] = value
    if not groups:
        for name, attr in (('keys', 'key_cache'), ('values', 'value_cache')):
            seq = getattr(kv_cache, attr, None)
            if isinstance(seq, (list, tuple)) and layer_idx < len(seq) and isinstance(seq[layer_idx], torch.Tensor):
                groups[name] = seq[layer_idx]
    if not groups:
        raise ValueError(f'Unable to locate cache tensors for layer {layer_idx}')
    return groups


def extract_exp_freq(kv_cache, freq_type: str = 'exp', prefill_len=None, dtype: str = 'bf16',
                     backend: str = 'traditional_kv') -> dict:
    """``{layer_idx: {"prefill_keys": [...], "decode_keys": [...], ...}}`` (or ``keys`` /
    ``values`` without ``prefill_len``) for every layer of the cache (reference: :271-296)."""
    if freq_type != 'exp':
        raise NotImplementedError("only freq_type='exp' feeds the float11 cache path")
    if backend != 'traditional_kv':
        raise NotImplementedError("only backend='traditional_kv' is provided")
    out = {}
    for layer_idx in range(len(kv_cache.layers)):
        pair = {}
        for name, tensor in _layer_tensor_groups(kv_cache, layer_idx).items():
            if prefill_len is not None:
                prefill, decode = _slice_prefill_decode(tensor, prefill_len)
                pair[f'prefill_{name}'] = get_exp_freq_list(prefill, dtype)
                pair[f'decode_{name}'] = get_exp_freq_list(decode, dtype)
            else:
                pair[name] = get_exp_freq_list(tensor, dtype)
        out[layer_idx] = pair
    return out


def merge_exp_freq(freq1: dict, freq2: dict) -> dict:
    """Bin-wise sum of two results of ``extract_exp_freq`` (reference: :298-307)."""
    return {k1: {k2: [a + b for a, b in zip(freq1[k1][k2], freq2[k1][k2])] for k2 in freq1[k1]} for k1 in freq1}

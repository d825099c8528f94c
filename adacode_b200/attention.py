"""Decode-step attention computed from the packed cache (``adacode_decode_attn``).

The reference rebuilds dense K and V on every ``Cache.update`` (``decode_impl:
'materialize_dense'``, float_cache_utils.py:1342) and lets the model's own attention read
them.  For a single new token that moves, per cached element, the packed bytes in, two dense
bytes out and two dense bytes in again.  The kernel behind this module reads the packed planes
once and never writes dense K/V.

The result is attention over the exact (lossless) cache with fp32 accumulation (for head_dim 128
the products run on the tensor cores and the probabilities are rounded to bf16 first), rounded
to bf16; it is *not* bit-identical to what a model's stock attention kernel produces from the
same dense K/V, because the order of the fp32 sums differs.  Token-for-token equality with an uncompressed
cache is only promised by the materialising path (``Float11Cache.update``).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from . import _lib
from .codec import _scratch_for, _stream_ptr, build_segment_table

_SEQ_TILE = 128
_MAX_SPLITS = 128

_workspaces: dict = {}


def _workspace(device: torch.device, need: int) -> torch.Tensor:
    ws = _workspaces.get(device)
    if ws is None or ws.numel() < need:
        ws = _workspaces[device] = torch.empty(need, dtype=torch.uint8, device=device)
    return ws


def decode_attention(query: torch.Tensor, key_segments: Sequence, value_segments: Sequence,
                     key_tail: Optional[torch.Tensor] = None, value_tail: Optional[torch.Tensor] = None,
                     scale: Optional[float] = None, n_splits: int = 0,
                     key_table: Optional[torch.Tensor] = None, value_table: Optional[torch.Tensor] = None,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``softmax(scale * q K^T) V`` for one query token per sequence.

    ``query`` is bf16 ``[B, Hq, D]`` (or ``[B, Hq, 1, D]``); ``key_segments`` / ``value_segments``
    are the packed 128-token segments of one layer in sequence order (``TiledCompressedTensor`` or
    ``SegmentRef``, any mix of windows and code lengths); ``key_tail`` / ``value_tail`` are the
    dense bf16 ``[B, Hkv, T, D]`` tokens that follow them (the cache's residual).  Every cached
    token is attended to.  Returns bf16 with the shape of ``query``.
    """
    squeeze = query.dim() == 4
    if squeeze:
        if query.shape[2] != 1:
            raise ValueError('decode_attention takes one query token per sequence')
        q = query[:, :, 0, :]
    else:
        q = query
    if q.dtype != torch.bfloat16 or q.dim() != 3:
        raise ValueError('query must be bf16 [B, Hq, D]')
    if q.stride(-1) != 1:
        q = q.contiguous()
    if len(key_segments) != len(value_segments):
        raise ValueError('key and value must hold the same number of packed segments')
    B, Hq, D = q.shape
    dev = q.device
    sc = _scratch_for(dev)
    n_seg = len(key_segments)
    tail_len = 0
    Hkv = None
    if n_seg:
        Bs, Hkv, T, Ds = key_segments[0].original_shape
        if (Bs, Ds) != (B, D) or T != _SEQ_TILE:
            raise ValueError(f'segments are {key_segments[0].original_shape}, query is {tuple(q.shape)}')
        if tuple(value_segments[0].original_shape) != (Bs, Hkv, T, Ds):
            raise ValueError('key and value segments differ in shape')
    if key_tail is not None and key_tail.shape[-2] > 0:
        if value_tail is None or value_tail.shape != key_tail.shape or value_tail.stride() != key_tail.stride():
            raise ValueError('key_tail and value_tail must share shape and strides')
        if key_tail.dtype != torch.bfloat16 or key_tail.stride(-1) != 1 or key_tail.dim() != 4:
            raise ValueError('tails must be bf16 [B, Hkv, T, D] with unit stride along D')
        if Hkv is None:
            Hkv = key_tail.shape[1]
        if (key_tail.shape[0], key_tail.shape[1], key_tail.shape[3]) != (B, Hkv, D):
            raise ValueError('tail shape does not match the query / segments')
        tail_len = int(key_tail.shape[2])
    if Hkv is None:
        raise ValueError('the cache is empty')
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if n_seg:
        if key_table is None:
            key_table = build_segment_table(key_segments, None, dev)
        if value_table is None:
            value_table = build_segment_table(value_segments, None, dev)
    L = _lib.lib()
    need = int(L.adacode_decode_attn_workspace_bytes(B, Hq, D, n_splits if n_splits > 0 else _MAX_SPLITS))
    ws = _workspace(dev, need)
    if out is None:
        out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device=dev)
    elif out.dtype != torch.bfloat16 or tuple(out.shape) != (B, Hq, D) or not out.is_contiguous():
        raise ValueError('out must be a contiguous bf16 [B, Hq, D] tensor')
    tb, th, ts = (key_tail.stride()[:3] if tail_len else (0, 0, 0))
    with torch.cuda.device(dev):
        rc = L.adacode_decode_attn(
            q.data_ptr(), q.stride(0), q.stride(1),
            key_table.data_ptr() if n_seg else None, value_table.data_ptr() if n_seg else None, n_seg,
            key_tail.data_ptr() if tail_len else None, value_tail.data_ptr() if tail_len else None, tail_len,
            tb, th, ts, B, Hq, Hkv, _SEQ_TILE, D, float(scale), out.data_ptr(), ws.data_ptr(), ws.numel(),
            int(n_splits), sc.status.data_ptr(), _stream_ptr(dev))
    _lib.check(rc, 'adacode_decode_attn')
    return out.unsqueeze(2) if squeeze else out

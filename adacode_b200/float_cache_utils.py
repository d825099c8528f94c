"""``float11`` KV cache for HF transformers on B200: ``float11Layer`` and ``Float11Cache``.

Drop-in for the reference's ``float_cache_utils.py`` in its ``segmented_tiled`` layout: same
constructor arguments, same ``update`` / ``get_seq_length`` / ``materialize_layer`` /
``get_layer_cache_view`` / ``get_memory`` / ``get_compress_params`` /
``synchronize_and_release`` surface, the same segment contents (window, code length and
bytes of every packed 128-token block) and the same counters after any sequence of updates.

What is different is how the work is done:
  * a prefill packs all its full blocks with ONE kernel launch straight from the (possibly
    strided) projection output, instead of one launch pair, eight torch ops and a host sync
    per block and a re-slice of the remaining prompt after every block
    (reference: float_cache_utils.py:1117-1140, :1173-1199);
  * the dense K/V handed to attention is produced by ONE unpack launch over a device-side
    segment table into a workspace, instead of one launch per segment plus ``torch.cat`` of
    everything (reference: :1245-1290);
  * the residual (not yet packed tail) lives in a preallocated buffer, not a chain of
    ``torch.cat`` results (reference: :869-881);
  * the exponent histogram of a staged block comes from a histogram kernel, not from packing
    the block and throwing the result away (reference: :1142-1159).

The adjuster state machine (when a proposal is made, when it is adopted, when it is dropped,
when blocks are staged, re-packed or packed late) follows the reference line by line in
meaning; the places are cited at each method.
"""
from __future__ import annotations

import time
import warnings
from typing import Any, Optional

import torch
from transformers import Cache
from transformers.cache_utils import DynamicLayer

from . import codec
from .codec import SegmentRef, TiledCompressedTensor

_SUPPORTED_LAYOUTS = ('segmented_tiled', 'legacy', 'tiled')
_LEGACY_BLOCK_GAPS = (8, 4, 8, 2)      # escape-base blocks of the flat layout: 128 x gap elements
_MAX_LAUNCH_ELEMS = 2 ** 31 - 1         # one pack launch (keys and values together) stays below this


def _segmented_state(segment_states: list) -> Optional[dict]:
    """Summary dict over a list of exported segment states
    (reference: float_cache_utils.py:72-97)."""
    if not segment_states:
        return None
    first = segment_states[0]
    batch_size, num_kv_heads, _, head_dim = tuple(first['original_shape'])
    seq_lens = [int(tuple(s['original_shape'])[-2]) for s in segment_states]
    return {
        'layout': 'segmented_tiled', 'kind': 'segmented_tiled', 'segments': list(segment_states),
        'num_segments': len(segment_states), 'segment_seq_lens': seq_lens,
        'logical_seq_len_total': sum(seq_lens),
        'original_shape': (batch_size, num_kv_heads, sum(seq_lens), head_dim),
        'seq_tile_size': first['seq_tile_size'], 'head_dim': first['head_dim'],
        'tile_head_dim': first['tile_head_dim'], 'tile_num_lanes': first['tile_num_lanes'],
        'num_kv_heads': first['num_kv_heads'],
        'num_sequence_tiles': sum(int(s.get('num_sequence_tiles', 0)) for s in segment_states),
        'device': first['device'], 'nbits': first['nbits'], 'left': first['left'], 'right': first['right'],
    }


class _DenseWorkspace:
    """Flat bf16 buffers, one per (device, slot), that hold the dense view of ONE layer at a
    time.  Every layer of a cache unpacks into the same memory, so the dense copy of the
    cache costs one layer, not all of them."""

    def __init__(self):
        self._bufs: dict = {}

    def view(self, device, slot: str, shape: tuple) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        key = (torch.device(device), slot)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(max(int(n * 1.25), 1 << 16), dtype=torch.bfloat16, device=device)
            self._bufs[key] = buf
        return buf[:n].view(shape)

    def release(self):
        self._bufs.clear()


_GLOBAL_WORKSPACE = _DenseWorkspace()


class _Residual:
    """The not-yet-packed tail of one tensor: a preallocated [B, H, capacity, D] buffer and a
    length.  ``None`` tensors in the reference correspond to ``length == 0`` here."""

    def __init__(self):
        self.buf: Optional[torch.Tensor] = None
        self.length = 0

    def tensor(self) -> Optional[torch.Tensor]:
        if self.buf is None or self.length == 0:
            return None
        return self.buf[:, :, : self.length]

    def _reserve(self, like: torch.Tensor, need: int, block: int) -> None:
        if self.buf is not None and self.buf.shape[2] >= need:
            return
        B, H, _, D = like.shape
        cap = max(2 * block, 1)
        while cap < need:
            cap *= 2
        new = torch.empty((B, H, cap, D), dtype=torch.bfloat16, device=like.device)
        if self.buf is not None and self.length:
            new[:, :, : self.length].copy_(self.buf[:, :, : self.length])
        self.buf = new

    def append(self, states: torch.Tensor, block: int) -> None:
        q = int(states.shape[-2])
        if q == 0:
            return
        self._reserve(states, self.length + q, block)
        self.buf[:, :, self.length: self.length + q].copy_(states)
        self.length += q

    def drop_front(self, count: int) -> None:
        """Forget the first ``count`` tokens, moving what follows to the front."""
        count = int(count)
        rest = self.length - count
        if rest > 0:
            if rest <= count:
                self.buf[:, :, :rest].copy_(self.buf[:, :, count: self.length])
            else:
                self.buf[:, :, :rest].copy_(self.buf[:, :, count: self.length].clone())
        self.length = max(rest, 0)

    def clear(self) -> None:
        self.buf = None
        self.length = 0


class float11Layer(DynamicLayer):
    """One decoder layer's lossless cache (reference: float_cache_utils.py:492-1553)."""

    def __init__(
        self,
        keys_right: Optional[int] = 0,
        values_right: Optional[int] = 0,
        keys_nbits: Optional[int] = 3,
        values_nbits: Optional[int] = 3,
        residual_length: int = 0,
        block_size: int = 128,
        layout: str = 'legacy',
        seq_tile_size: Optional[int] = None,
        auto_init_compress_params: bool = False,
        dense_workspace: str = 'shared',
    ):
        super().__init__()
        if layout not in _SUPPORTED_LAYOUTS:
            raise ValueError(f'layout={layout!r}: expected one of {_SUPPORTED_LAYOUTS}')
        if dense_workspace not in ('shared', 'layer'):
            raise ValueError("dense_workspace must be 'shared' or 'layer'")
        self.residual_length = residual_length
        self.block_size = int(block_size)
        self.layout = layout
        self.seq_tile_size = seq_tile_size if seq_tile_size is not None else block_size
        self.auto_init_compress_params = bool(auto_init_compress_params)
        self.compress_params_initialized = (
            keys_right is not None and values_right is not None
            and keys_nbits is not None and values_nbits is not None)
        if self.auto_init_compress_params and self.compress_params_initialized:
            raise ValueError('auto_init_compress_params expects compression parameters to be None.')
        if not self.auto_init_compress_params and not self.compress_params_initialized:
            raise ValueError('Compression parameters must be provided unless auto_init_compress_params is enabled.')
        self.keys_right, self.keys_nbits = keys_right, keys_nbits
        self.values_right, self.values_nbits = values_right, values_nbits
        self.new_keys_right, self.new_keys_nbits = keys_right, keys_nbits
        self.new_values_right, self.new_values_nbits = values_right, values_nbits
        self.cumulative_length = 0
        self.keys_update_times = 0
        self.values_update_times = 0
        self.keys_update_proposals = 0
        self.values_update_proposals = 0
        self.cache_device = None
        self.cache_dtype = None
        self.materialize_calls = 0
        self.materialize_cache_hits = 0
        self.materialize_time = 0.0
        self.prefill_reuse_hits = 0
        self.auto_init_compress_param_updates = 0
        # packed prefix: one entry per 128-token block, for keys and for values
        self._key_segments: list[SegmentRef] = []
        self._value_segments: list[SegmentRef] = []
        self._compressed_prefix_seq_len = 0
        self._compressed_block_flushes = 0
        self._compressed_tokens_flushed = 0
        # dense tail
        self._res_k = _Residual()
        self._res_v = _Residual()
        # adjuster bookkeeping (reference: :560-566)
        self._pending_adjust_recompress_start_segment: Optional[int] = None
        self._pending_dense_block_seq_len = 0
        self._pending_dense_block_key_params: Optional[tuple] = None
        self._pending_dense_block_value_params: Optional[tuple] = None
        self._pending_dense_block_needs_adjust_params = False
        self._adjust_recompresses = 0
        self._delayed_adjust_block_flushes = 0
        # dense materialisation
        self.dense_workspace = dense_workspace
        self._workspace = _GLOBAL_WORKSPACE if dense_workspace == 'shared' else _DenseWorkspace()
        self._tables: dict = {}            # 'k' / 'v' -> (n_segments, device table)
        self._mirror: dict = {}            # 'layer' mode: 'k' / 'v' -> [B, H, capacity, D] dense mirror
        self._mirror_valid: dict = {'k': 0, 'v': 0}   # tokens of the mirror that hold cache contents
        self._materialized_prefix_seq_len = 0
        self._cache_view_static: Optional[dict] = None
        self._cache_view_runtime: Optional[dict] = None
        self._compressed_prefix_ready_event = None
        self._compressed_prefix_ready_event_pending = False
        # optional callable applied to every histogram before the adjuster reads it (sharded caches
        # sum the histograms of all shards here)
        self.hist_reduce = None
        self._escape_fraction = (None, None)   # of the last packed span, keys and values
        self._host_hists = None                # (device K hist, host copy, device V hist, host copy) of the last pack

    # ------------------------------------------------------------------ reference-named views
    @property
    def residual_keys(self) -> Optional[torch.Tensor]:
        return self._res_k.tensor()

    @property
    def residual_values(self) -> Optional[torch.Tensor]:
        return self._res_v.tensor()

    @property
    def _compressed_prefix_key_segments(self) -> list:
        return [s.export_state() for s in self._key_segments]

    @property
    def _compressed_prefix_value_segments(self) -> list:
        return [s.export_state() for s in self._value_segments]

    def segment_params(self) -> list:
        """[(keys (right, nbits), values (right, nbits))] of every packed block, oldest first."""
        return [((k.right, k.nbits), (v.right, v.nbits)) for k, v in zip(self._key_segments, self._value_segments)]

    # ------------------------------------------------------------------ pickling
    def __getstate__(self):
        state = self.__dict__.copy()
        event = state.get('_compressed_prefix_ready_event')
        if state.get('_compressed_prefix_ready_event_pending') and event is not None:
            event.synchronize()
        state['_compressed_prefix_ready_event'] = None
        state['_compressed_prefix_ready_event_pending'] = False
        state['_tables'] = {}              # hold raw device addresses
        state['_workspace'] = None
        state['hist_reduce'] = None          # process groups do not pickle
        state['_mirror'] = {}
        state['_mirror_valid'] = {'k': 0, 'v': 0}
        state['_host_hists'] = None
        state['_cache_view_static'] = None
        state['_cache_view_runtime'] = None
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)
        self._workspace = _GLOBAL_WORKSPACE if self.dense_workspace == 'shared' else _DenseWorkspace()
        self._compressed_prefix_ready_event = None
        self._compressed_prefix_ready_event_pending = False

    # ------------------------------------------------------------------ parameter bookkeeping
    def _set_compress_params(self, keys_params, values_params, *, count_as_auto_init: bool = False) -> None:
        self.keys_right, self.keys_nbits = int(keys_params[0]), int(keys_params[1])
        self.values_right, self.values_nbits = int(values_params[0]), int(values_params[1])
        self.new_keys_right, self.new_keys_nbits = self.keys_right, self.keys_nbits
        self.new_values_right, self.new_values_nbits = self.values_right, self.values_nbits
        self.compress_params_initialized = True
        if count_as_auto_init:
            self.auto_init_compress_param_updates += 1

    def _ensure_compress_params_initialized(self, key_states, value_states) -> None:
        """reference: :584-607."""
        if self.compress_params_initialized:
            return
        if not self.auto_init_compress_params:
            raise RuntimeError('Compression parameters are not initialized.')
        k_hist = self._extract_exponent_histogram(key_states)
        v_hist = self._extract_exponent_histogram(value_states)
        if k_hist is None or v_hist is None:
            raise RuntimeError('Unable to initialize compression parameters from empty KV tensors.')
        both = codec.read_back(torch.stack([k_hist.to(torch.int32), v_hist.to(torch.int32)]))
        self._set_compress_params(codec.analysis_best_bits(both[0]), codec.analysis_best_bits(both[1]),
                                  count_as_auto_init=True)

    def _record_adjust_proposal(self, new_keys_params, new_values_params) -> None:
        """reference: :624-641 — a proposal counts when it differs from the previous proposal."""
        if (int(self.new_keys_right), int(self.new_keys_nbits)) != (int(new_keys_params[0]), int(new_keys_params[1])):
            self.keys_update_proposals += 1
        if (int(self.new_values_right), int(self.new_values_nbits)) != (
                int(new_values_params[0]), int(new_values_params[1])):
            self.values_update_proposals += 1

    def _record_effective_param_update(self, old_keys, old_values, new_keys, new_values) -> None:
        """reference: :643-662."""
        if (int(old_keys[0]), int(old_keys[1])) != (int(new_keys[0]), int(new_keys[1])):
            self.keys_update_times += 1
        if (int(old_values[0]), int(old_values[1])) != (int(new_values[0]), int(new_values[1])):
            self.values_update_times += 1

    def adjust_compressor(self, keys_exp_count, values_exp_count) -> None:
        """'legacy' / 'tiled' layouts: the windows proposed by the histograms of the blocks packed on
        an adjust step wait in ``new_*`` until the next adjust step adopts them; nothing already packed
        changes (reference: :664-669; there the call runs on a thread pool and is joined at the next
        adjust step, here it runs at once)."""
        new_keys = codec.analysis_best_bits(keys_exp_count)
        new_values = codec.analysis_best_bits(values_exp_count)
        self._record_adjust_proposal(new_keys, new_values)
        self.new_keys_right, self.new_keys_nbits = int(new_keys[0]), int(new_keys[1])
        self.new_values_right, self.new_values_nbits = int(new_values[0]), int(new_values[1])

    def has_pending_adjust_recompress(self) -> bool:
        return self._pending_adjust_recompress_start_segment is not None

    def has_pending_adjust_work(self) -> bool:
        return self._pending_adjust_recompress_start_segment is not None or self._pending_dense_block_needs_adjust_params

    def has_pending_dense_block(self) -> bool:
        return self._pending_dense_block_seq_len > 0

    def mark_adjust_recompress_start(self, start_segment: int) -> None:
        """reference: :680-690."""
        start_segment = max(0, int(start_segment))
        cur = self._pending_adjust_recompress_start_segment
        self._pending_adjust_recompress_start_segment = start_segment if cur is None else min(cur, start_segment)

    def mark_dense_block_pending(self, seq_len: int, key_params, value_params, needs_adjust_params: bool) -> None:
        """reference: :692-704 (the length accumulates if staged blocks are never applied)."""
        self._pending_dense_block_seq_len += int(seq_len)
        self._pending_dense_block_key_params = (int(key_params[0]), int(key_params[1]))
        self._pending_dense_block_value_params = (int(value_params[0]), int(value_params[1]))
        self._pending_dense_block_needs_adjust_params = bool(needs_adjust_params)

    # ------------------------------------------------------------------ residual
    def _active_residual_tensors(self):
        return self._res_k.tensor(), self._res_v.tensor()

    def _append_residual(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        self._res_k.append(key_states, self.block_size)
        self._res_v.append(value_states, self.block_size)

    @staticmethod
    def _extract_exponent_histogram(states: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """reference: :883-891."""
        if states is None or states.numel() == 0:
            return None
        return codec.exponent_hist(states)

    def _collect_adjust_hist_from_active_residual(self):
        k, v = self._active_residual_tensors()
        if k is None or v is None:
            return None, None
        return self._extract_exponent_histogram(k), self._extract_exponent_histogram(v)

    # ------------------------------------------------------------------ packing
    def _invalidate_dense(self) -> None:
        self._tables = {}
        self._materialized_prefix_seq_len = 0
        self._cache_view_static = None
        self._cache_view_runtime = None

    def _pack_span(self, key_states: torch.Tensor, value_states: torch.Tensor, need_adjust: bool):
        """Pack every full block of the two spans with the current windows and append the
        segments (reference: _flush_one_block / _compress_span / _append_compressed_prefix_span,
        :1117-1140, :993-1011, :1029-1056, applied to all blocks at once)."""
        if not self.compress_params_initialized:
            self._ensure_compress_params_initialized(key_states, value_states)
        if self.seq_tile_size != self.block_size:
            raise ValueError(
                'Tiled compressed path currently requires seq_tile_size == seq_len per compressed block, '
                f'got seq_tile_size={self.seq_tile_size}, seq_len={self.block_size}')
        if self.layout == 'tiled':
            # one unified state per tensor: a block of another code length cannot join it
            # (reference: _append_tiled_prefix_state, :277-283)
            for segs, nbits in ((self._key_segments, self.keys_nbits), (self._value_segments, self.values_nbits)):
                if segs and int(segs[0].nbits) != int(nbits):
                    raise ValueError('Tiled prefix append requires matching nbits, '
                                     f'got existing={int(segs[0].nbits)}, new={int(nbits)}')
        # keys and values go through one launch (two when their code lengths differ) and share one read
        # of their escape totals, status words and histograms; the escape buffers are sized from what
        # this layer's last span needed.  A launch covers fewer than 2**31 elements: longer spans are
        # packed in several launches, block range by block range.
        B, H, S, D = key_states.shape
        per_block = max(int(B * H * self.seq_tile_size * max(D, value_states.shape[-1])), 1)
        blocks_per_call = max(1, _MAX_LAUNCH_ELEMS // (2 * per_block))
        total_blocks = S // self.seq_tile_size
        k_hist = v_hist = kh_host = vh_host = None
        for b_lo in range(0, total_blocks, blocks_per_call):
            t_lo = b_lo * self.seq_tile_size
            t_hi = min(total_blocks, b_lo + blocks_per_call) * self.seq_tile_size
            ks, vs = key_states[:, :, t_lo:t_hi], value_states[:, :, t_lo:t_hi]
            nk, nv = ks.numel(), vs.numel()
            caps = tuple(None if f is None else int(n * f * 1.25) + 4096 for n, f in zip((nk, nv), self._escape_fraction))
            k_chunk, v_chunk, kh, vh, kh_h, vh_h = codec.pack_pair(
                ks, vs, (self.keys_right, self.keys_nbits), (self.values_right, self.values_nbits),
                self.seq_tile_size, need_hist=need_adjust, capacities=caps)
            self._escape_fraction = (k_chunk.n_escapes / max(nk, 1), v_chunk.n_escapes / max(nv, 1))
            if need_adjust:
                if k_hist is None:
                    k_hist, v_hist, kh_host, vh_host = kh, vh, kh_h, vh_h
                else:
                    k_hist, v_hist = k_hist + kh, v_hist + vh
                    kh_host, vh_host = kh_host + kh_h, vh_host + vh_h
            self._key_segments.extend(k_chunk.segments())
            self._value_segments.extend(v_chunk.segments())
        self._host_hists = (k_hist, kh_host, v_hist, vh_host) if need_adjust else None
        n_blocks = total_blocks
        tokens = n_blocks * self.seq_tile_size
        self._compressed_prefix_seq_len += tokens
        self._compressed_block_flushes += n_blocks
        self._compressed_tokens_flushed += tokens
        self._invalidate_dense()
        self._record_compressed_prefix_ready_event()
        return k_hist, v_hist

    def _record_compressed_prefix_ready_event(self) -> None:
        """reference: :1091-1104."""
        if self.cache_device is None or torch.device(self.cache_device).type != 'cuda' or \
                self._compressed_prefix_seq_len <= 0:
            self._compressed_prefix_ready_event = None
            self._compressed_prefix_ready_event_pending = False
            return
        with torch.cuda.device(self.cache_device):
            if self._compressed_prefix_ready_event is None:
                self._compressed_prefix_ready_event = torch.cuda.Event(blocking=False, interprocess=False)
            self._compressed_prefix_ready_event.record(torch.cuda.current_stream(self.cache_device))
        self._compressed_prefix_ready_event_pending = True

    def wait_for_compressed_prefix_ready(self, device=None) -> bool:
        """reference: :1106-1115."""
        if not self._compressed_prefix_ready_event_pending or self._compressed_prefix_ready_event is None:
            return False
        wait_device = self.cache_device if device is None else device
        if wait_device is None or torch.device(wait_device).type != 'cuda':
            return False
        with torch.cuda.device(wait_device):
            torch.cuda.current_stream(wait_device).wait_event(self._compressed_prefix_ready_event)
        self._compressed_prefix_ready_event_pending = False
        return True

    def _flush_full_blocks_from_residual(self, need_adjust: bool):
        """Pack all full blocks at the front of the residual (non-delayed flush)."""
        n_blocks = self._res_k.length // self.block_size
        if n_blocks == 0:
            return None, None, False
        tokens = n_blocks * self.block_size
        k_hist, v_hist = self._pack_span(self._res_k.buf[:, :, :tokens], self._res_v.buf[:, :, :tokens], need_adjust)
        self._res_k.drop_front(tokens)
        self._res_v.drop_front(tokens)
        return k_hist, v_hist, True

    def _stage_dense_block(self, collect_adjust_hist: bool):
        """A full block reached in decode stays dense until this layer's next update; only its
        histogram is taken now when an adjust step asks for it (reference: :1142-1159)."""
        k_hist = v_hist = None
        if collect_adjust_hist:
            if not self.compress_params_initialized:
                self._ensure_compress_params_initialized(*self._active_residual_tensors())
            k_hist = codec.exponent_hist(self._res_k.buf[:, :, : self.block_size])
            v_hist = codec.exponent_hist(self._res_v.buf[:, :, : self.block_size])
        self.mark_dense_block_pending(self.block_size, (self.keys_right, self.keys_nbits),
                                      (self.values_right, self.values_nbits), collect_adjust_hist)
        return k_hist, v_hist

    def _flush_ready_blocks(self, need_adjust: bool, delay_segmented_block: bool = False,
                            collect_adjust_hist: bool = False):
        """reference: :1161-1199."""
        if self._res_k.length < self.block_size:
            return None, None, False
        if not self.compress_params_initialized:
            self._ensure_compress_params_initialized(*self._active_residual_tensors())
        if delay_segmented_block:
            k_hist, v_hist = self._stage_dense_block(collect_adjust_hist)
            return k_hist, v_hist, False
        start_segment = len(self._key_segments) if need_adjust and self.layout == 'segmented_tiled' else None
        k_hist, v_hist, flushed = self._flush_full_blocks_from_residual(need_adjust)
        if start_segment is not None and k_hist is not None:
            self.mark_adjust_recompress_start(start_segment)
        return k_hist, v_hist, flushed

    # ------------------------------------------------------------------ adjuster
    def _update_adjust_params_from_hist(self, keys_exp_count, values_exp_count) -> bool:
        """reference: :902-938 (segmented_tiled branch): the proposal is stored; it replaces the
        staged block's windows when a block is staged, otherwise it waits in ``new_*``."""
        if keys_exp_count is None or values_exp_count is None:
            return False
        if self.hist_reduce is not None:
            keys_exp_count = self.hist_reduce(keys_exp_count)
            values_exp_count = self.hist_reduce(values_exp_count)
        cached = self._host_hists
        if cached is not None and self.hist_reduce is None and cached[0] is keys_exp_count and cached[2] is values_exp_count:
            k_host, v_host = cached[1], cached[3]        # came back with the pack's own read
        else:
            both = codec.read_back(torch.stack([keys_exp_count.to(torch.int32), values_exp_count.to(torch.int32)]))
            k_host, v_host = both[0], both[1]
        self._host_hists = None
        new_keys = codec.analysis_best_bits(k_host)
        new_values = codec.analysis_best_bits(v_host)
        if not self.compress_params_initialized:
            if not self.auto_init_compress_params:
                raise RuntimeError('Compression parameters are not initialized.')
            self._set_compress_params(new_keys, new_values, count_as_auto_init=True)
            return True
        self._record_adjust_proposal(new_keys, new_values)
        self.new_keys_right, self.new_keys_nbits = int(new_keys[0]), int(new_keys[1])
        self.new_values_right, self.new_values_nbits = int(new_values[0]), int(new_values[1])
        if self.has_pending_dense_block():
            self._pending_dense_block_key_params = (self.new_keys_right, self.new_keys_nbits)
            self._pending_dense_block_value_params = (self.new_values_right, self.new_values_nbits)
            self._pending_dense_block_needs_adjust_params = False
        return True

    def apply_pending_adjust_recompress_if_needed(self, keys_params, values_params) -> bool:
        """After a prefill packed with the calibrated windows, adopt the windows its own
        histogram proposes and, if they differ, unpack the segments and pack them again
        (reference: :706-793)."""
        start_segment = self._pending_adjust_recompress_start_segment
        self._pending_adjust_recompress_start_segment = None
        if start_segment is None:
            return False
        new_keys = (int(keys_params[0]), int(keys_params[1]))
        new_values = (int(values_params[0]), int(values_params[1]))
        old_keys = (self.keys_right, self.keys_nbits)
        old_values = (self.values_right, self.values_nbits)
        self._record_adjust_proposal(new_keys, new_values)
        self.new_keys_right, self.new_keys_nbits = new_keys
        self.new_values_right, self.new_values_nbits = new_values
        self.keys_right, self.keys_nbits = new_keys
        self.values_right, self.values_nbits = new_values
        if (old_keys, old_values) == (new_keys, new_values):
            return False
        self._record_effective_param_update(old_keys, old_values, new_keys, new_values)
        if start_segment >= len(self._key_segments):
            return False
        dense_k, dense_v = self._unpack_segment_range(start_segment)
        if dense_k is None or dense_k.shape[-2] == 0:
            return False
        self._key_segments = self._key_segments[:start_segment]
        self._value_segments = self._value_segments[:start_segment]
        self._compressed_prefix_seq_len = sum(int(s.original_shape[-2]) for s in self._key_segments)
        self._compressed_block_flushes = len(self._key_segments)
        self._compressed_tokens_flushed = self._compressed_prefix_seq_len
        self._invalidate_dense()
        # the unpacked span is a whole number of blocks: pack it again with the new windows;
        # the residual that was active stays behind it, untouched
        self._pack_span(dense_k, dense_v, need_adjust=False)
        self._adjust_recompresses += 1
        return True

    def apply_pending_dense_block_if_needed(self, keys_params=None, values_params=None) -> bool:
        """Pack the block staged at the previous update, with the windows captured (or proposed)
        when it was staged; this also overwrites any proposal still waiting in ``new_*``
        (reference: :795-856)."""
        pending_len = int(self._pending_dense_block_seq_len)
        if pending_len <= 0:
            return False
        if self._res_k.length < pending_len:
            return False
        if keys_params is None:
            keys_params = self._pending_dense_block_key_params
        if values_params is None:
            values_params = self._pending_dense_block_value_params
        if keys_params is None or values_params is None:
            return False
        self._pending_dense_block_seq_len = 0
        self._pending_dense_block_needs_adjust_params = False
        self._pending_dense_block_key_params = None
        self._pending_dense_block_value_params = None

        old_keys = (self.keys_right, self.keys_nbits)
        old_values = (self.values_right, self.values_nbits)
        self.new_keys_right, self.new_keys_nbits = int(keys_params[0]), int(keys_params[1])
        self.new_values_right, self.new_values_nbits = int(values_params[0]), int(values_params[1])
        self._record_adjust_proposal((self.new_keys_right, self.new_keys_nbits),
                                     (self.new_values_right, self.new_values_nbits))
        self.keys_right, self.keys_nbits = self.new_keys_right, self.new_keys_nbits
        self.values_right, self.values_nbits = self.new_values_right, self.new_values_nbits
        self._record_effective_param_update(old_keys, old_values, (self.keys_right, self.keys_nbits),
                                            (self.values_right, self.values_nbits))
        # only whole blocks inside the staged span are packed; a remainder stays at the front
        tokens = (pending_len // self.block_size) * self.block_size
        if tokens > 0:
            self._pack_span(self._res_k.buf[:, :, :tokens], self._res_v.buf[:, :, :tokens], need_adjust=False)
            self._res_k.drop_front(tokens)
            self._res_v.drop_front(tokens)
        self._delayed_adjust_block_flushes += 1
        return True

    # ------------------------------------------------------------------ dense materialisation
    def _segment_table(self, which: str, segments: list) -> torch.Tensor:
        cached = self._tables.get(which)
        if cached is not None and cached[0] == len(segments):
            return cached[1]
        table = codec.build_segment_table(segments, None, self.cache_device)
        self._tables[which] = (len(segments), table)
        return table

    def _unpack_segment_range(self, start: int):
        """Dense [B, H, n*block, D] tensors of segments[start:] (fresh tensors)."""
        ks, vs = self._key_segments[start:], self._value_segments[start:]
        if not ks:
            return None, None
        outs = []
        for segs in (ks, vs):
            B, H, T, D = segs[0].original_shape
            out = torch.empty((B, H, T * len(segs), D), dtype=torch.bfloat16, device=self.cache_device)
            codec.unpack_segments(segs, out)
            outs.append(out)
        return outs[0], outs[1]

    def _materialize_into_workspace(self):
        res_k, res_v = self._active_residual_tensors()
        res_len = 0 if res_k is None else int(res_k.shape[-2])
        prefix = self._compressed_prefix_seq_len
        total = prefix + res_len
        outs = []
        if self.dense_workspace == 'shared':
            # keys and values are decoded by one launch when they have one shape
            todo = []
            for which, segs in (('k', self._key_segments), ('v', self._value_segments)):
                B, H, _, D = segs[0].original_shape
                dense = self._workspace.view(self.cache_device, which, (B, H, total, D))
                todo.append((segs, dense, self._segment_table(which, segs)))
            codec.unpack_segments_multi(todo)
        for i, (which, segs, res) in enumerate((('k', self._key_segments, res_k), ('v', self._value_segments, res_v))):
            B, H, _, D = segs[0].original_shape
            if self.dense_workspace == 'shared':
                dense = todo[i][1]
            else:
                # per-layer mirror: lossless packing never changes a token's bits, so whatever was
                # written once stays valid; only blocks not yet present are decoded
                mirror = self._layer_mirror(which, (B, H, D), total)
                done = self._mirror_valid[which]
                if done < prefix:
                    first = done // self.seq_tile_size
                    offs = [i * self.seq_tile_size for i in range(first, len(segs))]
                    codec.unpack_segments(segs[first:], mirror, seq_offsets=offs)
                dense = mirror[:, :, :total]
                self._mirror_valid[which] = total
            if res_len:
                dense[:, :, prefix:total].copy_(res)
            outs.append(dense)
        return outs[0], outs[1]

    def _layer_mirror(self, which: str, bhd: tuple, total: int) -> torch.Tensor:
        buf = self._mirror.get(which)
        if buf is None or buf.shape[2] < total:
            B, H, D = bhd
            cap = max(2 * self.block_size, int(total * 1.5))
            new = torch.empty((B, H, cap, D), dtype=torch.bfloat16, device=self.cache_device)
            valid = self._mirror_valid.get(which, 0) if buf is not None else 0
            if valid:
                new[:, :, :valid].copy_(buf[:, :, :valid])
            self._mirror_valid[which] = valid
            self._mirror[which] = buf = new
        return buf

    def materialize_dense(self):
        """Dense (keys, values) of everything cached (reference: :1266-1290)."""
        begin = time.perf_counter()
        self.materialize_calls += 1
        if not self._key_segments:
            res_k, res_v = self._active_residual_tensors()
            self.materialize_time += time.perf_counter() - begin
            if res_k is None:
                return self._empty_states(), self._empty_states()
            return res_k, res_v
        if self._materialized_prefix_seq_len == int(self._compressed_prefix_seq_len) and self.layout != 'tiled':
            # no block was packed since the last call (reference: :1250-1256; its 'tiled' layout has no
            # cached prefix and never counts a hit)
            self.materialize_cache_hits += 1
        self._materialized_prefix_seq_len = int(self._compressed_prefix_seq_len)
        keys, values = self._materialize_into_workspace()
        self.materialize_time += time.perf_counter() - begin
        return keys, values

    def decode_attention(self, query: torch.Tensor, scale: Optional[float] = None, n_splits: int = 0) -> torch.Tensor:
        """Attention of one query token per sequence over everything this layer caches, read
        from the packed planes and the dense residual without rebuilding dense K/V.  The
        reference has no such path (its ``decode_impl`` is always ``'materialize_dense'``, :1342)."""
        from . import attention
        res_k, res_v = self._active_residual_tensors()
        if res_k is not None and res_k.stride() != res_v.stride():
            res_k, res_v = res_k.contiguous(), res_v.contiguous()
        ks, vs = self._key_segments, self._value_segments
        return attention.decode_attention(
            query, ks, vs, res_k, res_v, scale=scale, n_splits=n_splits,
            key_table=self._segment_table('k', ks) if ks else None,
            value_table=self._segment_table('v', vs) if vs else None)

    def _empty_states(self):
        if self.cache_device is None:
            return None
        return torch.empty((0,), device=self.cache_device, dtype=self.cache_dtype)

    # ------------------------------------------------------------------ introspection
    def get_cache_view(self) -> dict:
        """reference: :1331-1361."""
        if self.layout == 'segmented_tiled':
            key_meta = _segmented_state([s.export_decode_view() for s in self._key_segments])
            value_meta = _segmented_state([s.export_decode_view() for s in self._value_segments])
        elif self.layout == 'tiled':
            key_meta = self._unified_tiled_state(self._key_segments)
            value_meta = self._unified_tiled_state(self._value_segments)
        else:
            key_meta = value_meta = None           # the flat layout publishes no prefix metadata (reference: :1052-1066)
        res_k, res_v = self._active_residual_tensors()
        return {
            'layout': self.layout,
            'compressed_prefix_key': key_meta,
            'compressed_prefix_value': value_meta,
            'compressed_prefix_seq_len': self._compressed_prefix_seq_len,
            'closed_compressed_prefix_seq_len': self._compressed_prefix_seq_len,
            'block_size': self.block_size,
            'seq_tile_size': self.seq_tile_size,
            'decode_impl': 'materialize_dense',
            'residual_keys': res_k,
            'residual_values': res_v,
            'seq_length': self.cumulative_length,
            '_float11_layer': self,
        }

    # per-block states in the reference's own schemas, for consumers written against them
    @property
    def _compressed_prefix_key_blocks(self) -> list:
        return [self._legacy_block_state(s) for s in self._key_segments] if self.layout == 'legacy' else []

    @property
    def _compressed_prefix_value_blocks(self) -> list:
        return [self._legacy_block_state(s) for s in self._value_segments] if self.layout == 'legacy' else []

    @property
    def _compressed_prefix_key_state(self) -> Optional[dict]:
        return self._unified_tiled_state(self._key_segments) if self.layout == 'tiled' else None

    @property
    def _compressed_prefix_value_state(self) -> Optional[dict]:
        return self._unified_tiled_state(self._value_segments) if self.layout == 'tiled' else None

    @staticmethod
    def _legacy_block_state(seg) -> dict:
        """One packed block as ``CompressorBitMap.export_state`` gives it (compress_bitmap_merge.py:693-709):
        the planes are the segment's; ``block_base`` (inclusive escape count per 128 x gap elements) is
        counted from the code plane."""
        nbits, left, right = int(seg.nbits), int(seg.left), int(seg.right)
        n = int(seg.n_elements)
        ibs = 128 * _LEGACY_BLOCK_GAPS[nbits - 1]
        codes = seg.exp_data.reshape(-1)
        # codes of eight elements form one big-endian nbits-byte word
        words = codes.view(-1, nbits).to(torch.int64)
        g = torch.zeros(words.shape[0], dtype=torch.int64, device=codes.device)
        for i in range(nbits):
            g = (g << 8) | words[:, i]
        shifts = torch.arange(7, -1, -1, device=codes.device, dtype=torch.int64) * nbits
        is_escape = ((g.unsqueeze(1) >> shifts) & ((1 << nbits) - 1)) == 0          # [groups, 8] in element order
        flat = is_escape.reshape(-1)
        pad = (-n) % ibs
        if pad:
            flat = torch.cat([flat, torch.zeros(pad, dtype=torch.bool, device=flat.device)])
        block_base = torch.cumsum(flat.view(-1, ibs).sum(dim=1), dim=0)            # int64, as torch.cumsum gives it
        return {'right': right, 'nbits': nbits, 'left': left, 'left_nbits': left << 7, 'blocksize': 128,
                'invalid_block_size': ibs, 'device': seg.sign_mass_data.device,
                'original_shape': torch.Size(seg.original_shape), 'n_elements': n, 'n_exp_data': n * nbits // 8,
                'sign_mass_data': seg.sign_mass_data.reshape(-1), 'exp_data': codes,
                'invalid_exp': seg.invalid_exp, 'block_base': block_base}

    @staticmethod
    def _unified_tiled_state(segments) -> Optional[dict]:
        """All blocks of one tensor as ONE tiled state, planes in [b][h][tile] order with one running
        escape count over all tiles (what the reference's 'tiled' layout keeps, :249-329)."""
        if not segments:
            return None
        states = [s.export_state() for s in segments]
        first = states[0]
        B, H, T, D = tuple(first['original_shape'])
        nbits = int(first['nbits'])
        n = len(states)
        sm = torch.stack([st['sign_mass_data'].view(B, H, T * D) for st in states], dim=2).reshape(-1)
        cd = torch.stack([st['exp_data'].view(B, H, T * D * nbits // 8) for st in states], dim=2).reshape(-1)
        counts, chunks = [], []
        for st in states:
            base = st['tile_invalid_base'].to(torch.int64)
            c = base.clone()
            c[1:] = base[1:] - base[:-1]
            counts.append(c.view(B, H))
            chunks.append(list(torch.split(st['invalid_exp'], [int(v) for v in c.tolist()])))
        merged_counts = torch.stack(counts, dim=2).reshape(-1)
        esc = [chunks[j][bh] for bh in range(B * H) for j in range(n)]
        out = dict(first)
        out.update(sign_mass_data=sm, exp_data=cd,
                   invalid_exp=torch.cat(esc) if esc else first['invalid_exp'],
                   tile_invalid_base=torch.cumsum(merged_counts, dim=0).to(torch.int32),
                   original_shape=(B, H, T * n, D), num_sequence_tiles=n,
                   n_elements=sum(int(st['n_elements']) for st in states), kind='tiled_decode')
        return out

    def get_memory(self) -> dict:
        """reference: :1363-1498 (segmented_tiled branch).  Bytes are logical bytes of the packed
        streams plus the dense residual, which counts on both sides."""
        compressed = original = 0
        k_ratio = v_ratio = 0.0
        for k, v in zip(self._key_segments, self._value_segments):
            km, vm = k.get_memory(), v.get_memory()
            if self.layout == 'legacy':
                for seg, mem in ((k, km), (v, vm)):
                    B, H = int(seg.original_shape[0]), int(seg.original_shape[1])
                    blocks = -(-seg.n_elements // (128 * _LEGACY_BLOCK_GAPS[int(seg.nbits) - 1]))
                    mem['compressed_memory'] += 8 * blocks - 4 * B * H      # int64 bases (torch.cumsum promotes)
            compressed += km['compressed_memory'] + vm['compressed_memory']
            original += km['original_memory'] + vm['original_memory']
            k_ratio += k.n_escapes / k.n_elements if k.n_elements else 0.0
            v_ratio += v.n_escapes / v.n_elements if v.n_elements else 0.0
        res_k, res_v = self._active_residual_tensors()
        if res_k is not None:
            res_bytes = res_k.numel() * res_k.element_size() + res_v.numel() * res_v.element_size()
            compressed += res_bytes
            original += res_bytes
        n = len(self._key_segments)
        if n > 0:
            k_ratio /= n
            v_ratio /= n
        res_len = 0 if res_k is None else int(res_k.shape[-2])
        return {
            'compressed_memory': compressed,
            'original_memory': original,
            'keys_outlier_ratios': k_ratio,
            'values_outlier_ratios': v_ratio,
            'keys_update_times': self.keys_update_times,
            'values_update_times': self.values_update_times,
            'keys_update_proposals': self.keys_update_proposals,
            'values_update_proposals': self.values_update_proposals,
            'materialize_calls': self.materialize_calls,
            'materialize_cache_hits': self.materialize_cache_hits,
            'materialize_time': self.materialize_time,
            'stored_compressed_prefix_seq_len': self._compressed_prefix_seq_len,
            'stored_residual_seq_len': res_len,
            'compressed_block_flushes': self._compressed_block_flushes,
            'compressed_tokens_flushed': self._compressed_tokens_flushed,
            'residual_tokens_kept': res_len,
            'stored_compressed_block_count': 0 if self.block_size <= 0 else self._compressed_tokens_flushed // self.block_size,
            'prefill_reuse_hits': self.prefill_reuse_hits,
            'adjust_recompresses': self._adjust_recompresses,
            'delayed_adjust_block_flushes': self._delayed_adjust_block_flushes,
        }

    # ------------------------------------------------------------------ update
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, need_adjust: bool = False,
               cache_kwargs: Optional[dict] = None) -> dict:
        """reference: :1500-1550."""
        self.cumulative_length += key_states.shape[-2]
        first_update = not self.is_initialized
        if first_update:
            self.lazy_initialization(key_states, value_states)
            self.cache_device = key_states.device
            self.cache_dtype = key_states.dtype
        if need_adjust and self.compress_params_initialized and not self.has_pending_adjust_work():
            self.keys_right, self.keys_nbits = self.new_keys_right, self.new_keys_nbits
            self.values_right, self.values_nbits = self.new_values_right, self.new_values_nbits

        q_len = key_states.shape[-2]
        prefill_fastpath = q_len > 1 and first_update
        segmented = self.layout == 'segmented_tiled'
        if key_states.dtype != torch.bfloat16:
            key_states = key_states.to(torch.bfloat16)
        if value_states.dtype != torch.bfloat16:
            value_states = value_states.to(torch.bfloat16)

        if prefill_fastpath and self._res_k.length == 0:
            # all full blocks go from the projection output to packed planes in one launch;
            # only the tail (< block_size tokens) is copied into the residual buffer
            n_full = (q_len // self.block_size) * self.block_size
            keys_exp_count = values_exp_count = None
            flushed_any = False
            if n_full > 0:
                if not self.compress_params_initialized:
                    self._ensure_compress_params_initialized(key_states, value_states)
                start_segment = len(self._key_segments) if need_adjust and segmented else None
                keys_exp_count, values_exp_count = self._pack_span(
                    key_states[:, :, :n_full], value_states[:, :, :n_full], need_adjust)
                flushed_any = True
                if start_segment is not None and keys_exp_count is not None:
                    self.mark_adjust_recompress_start(start_segment)
            if n_full < q_len:
                self._append_residual(key_states[:, :, n_full:], value_states[:, :, n_full:])
        else:
            self._append_residual(key_states, value_states)
            keys_exp_count, values_exp_count, flushed_any = self._flush_ready_blocks(
                need_adjust=need_adjust,
                delay_segmented_block=segmented and not prefill_fastpath,
                collect_adjust_hist=segmented and need_adjust and not prefill_fastpath,
            )
        if segmented and need_adjust and keys_exp_count is None:
            keys_exp_count, values_exp_count = self._collect_adjust_hist_from_active_residual()
        if segmented and need_adjust:
            if prefill_fastpath and flushed_any:
                self.mark_adjust_recompress_start(0)
            self._update_adjust_params_from_hist(keys_exp_count, values_exp_count)

        if prefill_fastpath:
            self.prefill_reuse_hits += 1
            dense_keys, dense_values = key_states, value_states
        elif cache_kwargs is not None and cache_kwargs.get('float11_skip_materialize', False):
            dense_keys = dense_values = None      # the caller attends to the packed planes directly
        else:
            dense_keys, dense_values = self.materialize_dense()
        return {
            'key_states': dense_keys,
            'value_states': dense_values,
            'keys_exp_count': keys_exp_count,
            'values_exp_count': values_exp_count,
        }

    def get_seq_length(self) -> int:
        return self.cumulative_length

    def release(self) -> None:
        """Drop every tensor this layer holds (reference: Float11Cache.synchronize_and_release,
        :1781-1814)."""
        self._res_k.clear()
        self._res_v.clear()
        self._key_segments = []
        self._value_segments = []
        self._compressed_prefix_seq_len = 0
        self._compressed_block_flushes = 0
        self._compressed_tokens_flushed = 0
        self._pending_adjust_recompress_start_segment = None
        self._pending_dense_block_seq_len = 0
        self._pending_dense_block_key_params = None
        self._pending_dense_block_value_params = None
        self._pending_dense_block_needs_adjust_params = False
        self._adjust_recompresses = 0
        self._delayed_adjust_block_flushes = 0
        self._compressed_prefix_ready_event = None
        self._compressed_prefix_ready_event_pending = False
        self._invalidate_dense()
        self._mirror = {}
        self._mirror_valid = {'k': 0, 'v': 0}
        if self.dense_workspace != 'shared':
            self._workspace.release()


class Float11Cache(Cache):
    """HF ``Cache`` whose layers are ``float11Layer`` (reference: float_cache_utils.py:1556-1814).

    ``hist_reduce`` (optional callable, e.g. ``sharding.HistogramAllReduce``) and
    ``dense_workspace`` are the arguments the reference does not have.  ``dense_workspace``: ``'shared'`` (default)
    unpacks each layer into one workspace shared by all layers, so the K/V returned by
    ``update`` are valid until the next layer's ``update``; ``'layer'`` keeps an append-only
    dense mirror per layer, as the reference effectively does.
    """

    def __init__(
        self,
        config,
        right,
        exp_bits,
        need_adjust: bool = False,
        update_steps: int = 64,
        residual_length: int = 0,
        block_size: int = 128,
        layout: str = 'legacy',
        seq_tile_size: Optional[int] = None,
        auto_init_compress_params: bool = False,
        dense_workspace: str = 'shared',
        hist_reduce=None,
    ):
        config = config.get_text_config(decoder=True)
        auto_init_compress_params = bool(auto_init_compress_params)
        common = dict(residual_length=residual_length, block_size=block_size, layout=layout,
                      seq_tile_size=seq_tile_size, dense_workspace=dense_workspace)
        n_layers = config.num_hidden_layers
        if auto_init_compress_params:
            if right is not None or exp_bits is not None:
                raise ValueError('auto_init_compress_params expects right and exp_bits to be None.')
            layers = [float11Layer(None, None, None, None, auto_init_compress_params=True, **common)
                      for _ in range(n_layers)]
        elif right is None or exp_bits is None:
            raise ValueError('right and exp_bits are required unless auto_init_compress_params is enabled.')
        elif isinstance(right, int):
            layers = [float11Layer(right, right, exp_bits, exp_bits, **common) for _ in range(n_layers)]
        else:
            layers = [float11Layer(right[i][0], right[i][1], exp_bits[i][0], exp_bits[i][1], **common)
                      for i in range(n_layers)]
        for layer in layers:
            layer.hist_reduce = hist_reduce
        self._init_adjust_schedule(need_adjust, update_steps, block_size, layout)
        self.peak_mem = 0
        self._fused_decode = False         # set by hf_attention.fused_decode
        self.layout = layout
        self.seq_tile_size = seq_tile_size if seq_tile_size is not None else block_size
        self.auto_init_compress_params = auto_init_compress_params
        super().__init__(layers=layers)

    def _init_adjust_schedule(self, need_adjust, update_steps, block_size, layout) -> None:
        """reference: :1623-1642 — with the adjuster on, the period is rounded up to a multiple of
        the block size so that adjust steps coincide with the steps at which blocks fill."""
        self.steps = 0
        self.need_adjust = bool(need_adjust and update_steps != 0)
        self.update_steps = int(update_steps) if self.need_adjust else 0
        self._pending_adjusts: dict = {}
        self._segmented_adjust = self.need_adjust and layout == 'segmented_tiled'
        if self._segmented_adjust:
            steps_int = max(1, int(update_steps))
            block_int = max(1, int(block_size))
            self.update_steps = ((steps_int + block_int - 1) // block_int) * block_int
            if int(update_steps) != int(self.update_steps):
                warnings.warn(
                    'segmented_tiled adjuster rounds kv_adjust_update_steps up to a block_size multiple: '
                    f'{int(update_steps)} -> {int(self.update_steps)}.', RuntimeWarning)

    def __getstate__(self):
        state = self.__dict__.copy()
        state['_pending_adjusts'] = {}
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)
        self._pending_adjusts = {}

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[dict] = None):
        """reference: :1657-1698."""
        if self.layer_class_to_replicate is not None:
            while len(self.layers) <= layer_idx:
                self.layers.append(self.layer_class_to_replicate())
        layer = self.layers[layer_idx]
        if self._segmented_adjust:
            if layer.has_pending_adjust_recompress():
                layer.apply_pending_adjust_recompress_if_needed(
                    (layer.new_keys_right, layer.new_keys_nbits),
                    (layer.new_values_right, layer.new_values_nbits))
            elif layer.has_pending_dense_block() and not layer.has_pending_adjust_work():
                layer.apply_pending_dense_block_if_needed()
        need_adjust = self.need_adjust and self.steps % self.update_steps == 0
        fused = getattr(self, '_fused_decode', False) and key_states.shape[-2] == 1 and layer.is_initialized
        if fused:
            # hf_attention.fused_decode: the step's attention reads the packed planes itself
            cache_kwargs = dict(cache_kwargs or {}, float11_skip_materialize=True)
        result = layer.update(key_states, value_states, need_adjust, cache_kwargs)
        if need_adjust and not self._segmented_adjust and result['keys_exp_count'] is not None:
            # 'legacy' / 'tiled' layouts: the proposal waits for the next adjust step (reference: :1683-1693)
            both = codec.read_back(torch.stack([result['keys_exp_count'].to(torch.int32),
                                                result['values_exp_count'].to(torch.int32)]))
            layer.adjust_compressor(both[0], both[1])
        if layer_idx == len(self.layers) - 1:
            self.steps += 1
        if fused:
            return key_states, value_states
        return result['key_states'], result['value_states']

    def decode_attention(self, query: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
                         layer_idx: int, scale: Optional[float] = None, n_splits: int = 0) -> torch.Tensor:
        """One decode step of one layer without dense K/V: append the new token's ``key_states``
        / ``value_states`` ([B, Hkv, 1, D]) exactly as ``update`` does (same packing schedule and
        adjuster steps), then return ``softmax(scale * q K^T) V`` for ``query`` ([B, Hq, 1, D] or
        [B, Hq, D]) over the whole cache, computed from the packed planes.  Results are fp32
        attention rounded to bf16; they are close to, not bit-identical with, what a model's own
        attention kernel gives on the dense K/V that ``update`` returns."""
        if key_states.shape[-2] != 1:
            raise ValueError('decode_attention appends exactly one token per sequence; use update() for prefill')
        self.update(key_states, value_states, layer_idx, {'float11_skip_materialize': True})
        return self.layers[layer_idx].decode_attention(query, scale=scale, n_splits=n_splits)

    def get_layer_cache_view(self, layer_idx: int):
        return self.layers[layer_idx].get_cache_view()

    def materialize_layer(self, layer_idx: int):
        return self.layers[layer_idx].materialize_dense()

    _SUMMED = (
        'keys_update_times', 'values_update_times', 'keys_update_proposals', 'values_update_proposals',
        'materialize_calls', 'materialize_cache_hits', 'materialize_time', 'stored_compressed_prefix_seq_len',
        'stored_residual_seq_len', 'compressed_block_flushes', 'compressed_tokens_flushed', 'residual_tokens_kept',
        'stored_compressed_block_count', 'prefill_reuse_hits', 'adjust_recompresses', 'delayed_adjust_block_flushes',
    )

    def get_memory(self) -> dict:
        """reference: :1706-1755 (memory in GiB, outlier ratios averaged over layers)."""
        total: dict = {'kv_compressed_memory': 0, 'kv_original_memory': 0}
        total.update({k: 0 for k in self._SUMMED})
        total['materialize_time'] = 0.0
        total['keys_outlier_ratios'] = 0.0
        total['values_outlier_ratios'] = 0.0
        for layer in self.layers:
            m = layer.get_memory()
            total['kv_compressed_memory'] += m['compressed_memory']
            total['kv_original_memory'] += m['original_memory']
            for k in self._SUMMED:
                total[k] += m[k]
            total['keys_outlier_ratios'] += m['keys_outlier_ratios']
            total['values_outlier_ratios'] += m['values_outlier_ratios']
        total['keys_outlier_ratios'] /= len(self.layers)
        total['values_outlier_ratios'] /= len(self.layers)
        total['kv_compressed_memory'] /= 1024 ** 3
        total['kv_original_memory'] /= 1024 ** 3
        return total

    def get_compress_params(self) -> dict:
        """reference: :1757-1774."""
        return {
            'kv_auto_init_compress_params': bool(self.auto_init_compress_params),
            'kv_compress_params_initialized_layers': sum(int(l.compress_params_initialized) for l in self.layers),
            'kv_auto_init_compress_param_updates': sum(int(l.auto_init_compress_param_updates) for l in self.layers),
            'kv_current_rights': [
                None if not l.compress_params_initialized else (int(l.keys_right), int(l.values_right))
                for l in self.layers],
            'kv_current_nbits': [
                None if not l.compress_params_initialized else (int(l.keys_nbits), int(l.values_nbits))
                for l in self.layers],
        }

    def synchronize_and_release(self) -> None:
        """reference: :1776-1814."""
        self._pending_adjusts.clear()
        for layer in self.layers:
            layer.release()

"""``mla_float11``: the float11 cache for DeepSeek-style MLA latent caches.

Drop-in for the reference's ``mla_float_cache_utils.py``.  An MLA attention layer caches, per
token, one compressed KV latent (``kv_lora_rank`` dims) and one decoupled RoPE key
(``qk_rope_head_dim`` dims), both shaped [batch, 1, seq, dim].

  * ``compress_rope=True`` (default): latent and rope key go through ``Float11Cache`` as the
    "keys" and "values" tensors, each with its own window and code length
    (reference: mla_float_cache_utils.py:505-517, :605-606).
  * ``compress_rope=False``: only the latent is packed; the rope key stays dense.  Blocks are
    packed as soon as they fill (no staging), and the adjuster result is consumed at the
    layer's next update (reference: ``MLALatentFloat11DenseRopeLayer``, :45-445, and
    ``MLAFloat11Cache.update``, :597-641).  The reference packs the latent twice (once with the
    "values" window) and discards one copy; here it is packed once and the accounting that
    depended on the duplicate is reproduced.
"""
from __future__ import annotations

import time
import warnings
from typing import Any, Optional

import torch
from transformers import Cache

from . import codec
from .float_cache_utils import Float11Cache, _Residual, float11Layer


def _component_pairs(num_layers, first_right, second_right, first_nbits, second_nbits):
    rights = [[int(first_right), int(second_right)] for _ in range(num_layers)]
    nbits = [[int(first_nbits), int(second_nbits)] for _ in range(num_layers)]
    return rights, nbits


def _normalize_component_pairs(value, num_layers: int, name: str):
    """reference: :32-42."""
    if isinstance(value, int):
        return [[int(value), int(value)] for _ in range(num_layers)]
    if len(value) != num_layers:
        raise ValueError(f'{name} must have {num_layers} layer entries, got {len(value)}.')
    out = []
    for layer_idx, pair in enumerate(value):
        if not isinstance(pair, (list, tuple)) or len(pair) != 2:
            raise ValueError(f'{name}[{layer_idx}] must be a pair for latent/rope, got {pair!r}.')
        out.append([int(pair[0]), int(pair[1])])
    return out


class MLALatentFloat11DenseRopeLayer(float11Layer):
    """Latent packed, rope key dense (reference: mla_float_cache_utils.py:45-445)."""

    def __init__(self, latent_right: int = 127, latent_nbits: int = 4, residual_length: int = 0,
                 block_size: int = 128, layout: str = 'segmented_tiled', seq_tile_size: Optional[int] = None,
                 dense_workspace: str = 'shared'):
        super().__init__(keys_right=latent_right, values_right=latent_right, keys_nbits=latent_nbits,
                         values_nbits=latent_nbits, residual_length=residual_length, block_size=block_size,
                         layout=layout, seq_tile_size=seq_tile_size, dense_workspace=dense_workspace)
        self._rope_prefix = _Residual()          # append-only dense rope keys of the packed prefix

    # the second residual tensor is the rope key
    @property
    def residual_rope(self) -> Optional[torch.Tensor]:
        return self._res_v.tensor()

    @property
    def _dense_rope_prefix_seq_len(self) -> int:
        return self._rope_prefix.length

    @property
    def _dense_rope_prefix_blocks(self) -> list:
        t = self._rope_prefix.tensor()
        if t is None:
            return []
        return [t[:, :, i: i + self.block_size] for i in range(0, self._rope_prefix.length, self.block_size)]

    def _pack_span(self, key_states: torch.Tensor, value_states: torch.Tensor, need_adjust: bool):
        """Pack the latent span; keep the matching rope span dense.  Both histograms returned are
        the latent's (reference: :83-89, :131-160)."""
        if self.seq_tile_size != self.block_size:
            raise ValueError(
                'Tiled compressed path currently requires seq_tile_size == seq_len per compressed block, '
                f'got seq_tile_size={self.seq_tile_size}, seq_len={self.block_size}')
        chunk, hist = codec.pack_blocks(key_states, self.keys_right, self.keys_nbits, self.seq_tile_size,
                                        need_hist=need_adjust)
        if self.values_nbits not in (1, 2, 3, 4):
            # the reference packs the latent a second time with the "values" window and would fail here
            raise ValueError(f'Tiled compressed path supports nbits in (1, 2, 3, 4), got {self.values_nbits}')
        segs = chunk.segments()
        self._key_segments.extend(segs)
        self._value_segments.extend(segs)          # the duplicate the reference accounts for
        self._rope_prefix.append(value_states, self.block_size)
        tokens = chunk.n_blocks * self.seq_tile_size
        self._compressed_prefix_seq_len += tokens
        self._compressed_block_flushes += chunk.n_blocks
        self._compressed_tokens_flushed += tokens
        self._invalidate_dense()
        self._record_compressed_prefix_ready_event()
        return hist, hist

    def _flush_all_available_spans(self, need_adjust: bool):
        """reference: :162-185 — every full block is packed at once, also during decode."""
        n_blocks = self._res_k.length // self.block_size
        if n_blocks == 0:
            return None, None, False
        start_segment = len(self._key_segments) if need_adjust else None
        tokens = n_blocks * self.block_size
        k_hist, v_hist = self._pack_span(self._res_k.buf[:, :, :tokens], self._res_v.buf[:, :, :tokens], need_adjust)
        self._res_k.drop_front(tokens)
        self._res_v.drop_front(tokens)
        if start_segment is not None and k_hist is not None:
            self.mark_adjust_recompress_start(start_segment)
        return k_hist, v_hist, True

    def apply_pending_adjust_recompress_if_needed(self, keys_params, values_params) -> bool:
        """reference: :191-290 — the latent's proposal is used for both windows."""
        start_segment = self._pending_adjust_recompress_start_segment
        self._pending_adjust_recompress_start_segment = None
        if start_segment is None:
            return False
        new = (int(keys_params[0]), int(keys_params[1]))
        old_keys = (self.keys_right, self.keys_nbits)
        old_values = (self.values_right, self.values_nbits)
        self._record_adjust_proposal(new, new)
        self.new_keys_right, self.new_keys_nbits = new
        self.new_values_right, self.new_values_nbits = new
        self.keys_right, self.keys_nbits = new
        self.values_right, self.values_nbits = new
        if (old_keys, old_values) == (new, new):
            return False
        self._record_effective_param_update(old_keys, old_values, new, new)
        if start_segment >= len(self._key_segments):
            return False
        segs = self._key_segments[start_segment:]
        B, H, T, D = segs[0].original_shape
        latent = torch.empty((B, H, T * len(segs), D), dtype=torch.bfloat16, device=self.cache_device)
        codec.unpack_segments(segs, latent)
        rope_from = start_segment * self.block_size
        rope = self._rope_prefix.buf[:, :, rope_from: self._rope_prefix.length].clone()
        if latent.shape[-2] == 0 or rope.shape[-2] == 0:
            return False
        self._key_segments = self._key_segments[:start_segment]
        self._value_segments = self._value_segments[:start_segment]
        self._rope_prefix.length = rope_from
        self._compressed_prefix_seq_len = sum(int(s.original_shape[-2]) for s in self._key_segments)
        self._compressed_block_flushes = len(self._key_segments)
        self._compressed_tokens_flushed = self._compressed_prefix_seq_len
        self._invalidate_dense()
        self._pack_span(latent, rope, need_adjust=False)
        self._adjust_recompresses += 1
        return True

    def apply_pending_dense_block_if_needed(self, keys_params=None, values_params=None) -> bool:
        return super().apply_pending_dense_block_if_needed(keys_params, keys_params)

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, need_adjust: bool = False,
               cache_kwargs: Optional[dict] = None) -> dict:
        """reference: :307-357."""
        self.cumulative_length += key_states.shape[-2]
        first_update = not self.is_initialized
        if first_update:
            self.lazy_initialization(key_states, value_states)
            self.cache_device = key_states.device
            self.cache_dtype = key_states.dtype
        if need_adjust and not self.has_pending_adjust_work():
            self.keys_right, self.keys_nbits = self.new_keys_right, self.new_keys_nbits
            self.values_right, self.values_nbits = self.new_values_right, self.new_values_nbits
        q_len = key_states.shape[-2]
        prefill_fastpath = q_len > 1 and first_update
        if key_states.dtype != torch.bfloat16:
            key_states = key_states.to(torch.bfloat16)
        if value_states.dtype != torch.bfloat16:
            value_states = value_states.to(torch.bfloat16)

        if prefill_fastpath and self._res_k.length == 0:
            n_full = (q_len // self.block_size) * self.block_size
            keys_exp_count = values_exp_count = None
            flushed_any = False
            if n_full > 0:
                start_segment = len(self._key_segments) if need_adjust else None
                keys_exp_count, values_exp_count = self._pack_span(
                    key_states[:, :, :n_full], value_states[:, :, :n_full], need_adjust)
                flushed_any = True
                if start_segment is not None and keys_exp_count is not None:
                    self.mark_adjust_recompress_start(start_segment)
            if n_full < q_len:
                self._append_residual(key_states[:, :, n_full:], value_states[:, :, n_full:])
        else:
            self._append_residual(key_states, value_states)
            keys_exp_count, values_exp_count, flushed_any = self._flush_all_available_spans(need_adjust)
        if need_adjust and keys_exp_count is None:
            keys_exp_count, values_exp_count = self._collect_adjust_hist_from_active_residual()
        if need_adjust:
            if prefill_fastpath and flushed_any:
                self.mark_adjust_recompress_start(0)
            self._update_adjust_params_from_hist(keys_exp_count, values_exp_count)
        if prefill_fastpath:
            self.prefill_reuse_hits += 1
            dense_keys, dense_values = key_states, value_states
        else:
            dense_keys, dense_values = self.materialize_dense()
        return {'key_states': dense_keys, 'value_states': dense_values,
                'keys_exp_count': keys_exp_count, 'values_exp_count': values_exp_count}

    def _materialize_rope(self) -> Optional[torch.Tensor]:
        """reference: :359-382."""
        prefix = self._rope_prefix.tensor()
        res = self._res_v.tensor()
        if prefix is None:
            return res
        if res is None:
            return prefix
        return torch.cat([prefix, res], dim=-2)

    def materialize_dense(self):
        """reference: :384-408."""
        begin = time.perf_counter()
        self.materialize_calls += 1
        res_latent = self._res_k.tensor()
        if not self._key_segments:
            latent = res_latent if res_latent is not None else self._empty_states()
        else:
            if self._materialized_prefix_seq_len == int(self._compressed_prefix_seq_len):
                self.materialize_cache_hits += 1
            self._materialized_prefix_seq_len = int(self._compressed_prefix_seq_len)
            segs = self._key_segments
            B, H, _, D = segs[0].original_shape
            prefix = self._compressed_prefix_seq_len
            total = prefix + self._res_k.length
            if self.dense_workspace == 'shared':
                latent = self._workspace.view(self.cache_device, 'k', (B, H, total, D))
                codec.unpack_segments(segs, latent, table=self._segment_table('k', segs))
            else:
                mirror = self._layer_mirror('k', (B, H, D), total)
                done = self._mirror_valid['k']
                if done < prefix:
                    first = done // self.seq_tile_size
                    offs = [i * self.seq_tile_size for i in range(first, len(segs))]
                    codec.unpack_segments(segs[first:], mirror, seq_offsets=offs)
                latent = mirror[:, :, :total]
                self._mirror_valid['k'] = total
            if res_latent is not None:
                latent[:, :, prefix:total].copy_(res_latent)
        rope = self._materialize_rope()
        if rope is None:
            rope = self._empty_states()
        self.materialize_time += time.perf_counter() - begin
        return latent, rope

    def get_cache_view(self) -> dict:
        """reference: :410-417."""
        view = super().get_cache_view()
        view['layout'] = f'{self.layout}_mla_latent_dense_rope'
        view['compressed_prefix_value'] = None
        view['residual_values'] = self.residual_rope
        view['dense_rope_prefix_blocks'] = self._dense_rope_prefix_blocks
        view['dense_rope_prefix_seq_len'] = self._dense_rope_prefix_seq_len
        return view

    def get_memory(self) -> dict:
        """reference: :419-438 — the packed latent was counted twice by the base class."""
        info = super().get_memory()
        res_latent, res_rope = self._res_k.tensor(), self._res_v.tensor()
        residual_latent = 0 if res_latent is None else res_latent.numel() * res_latent.element_size()
        residual_rope = 0 if res_rope is None else res_rope.numel() * res_rope.element_size()
        residual = residual_latent + residual_rope
        rope_prefix = self._rope_prefix.tensor()
        rope_prefix_bytes = 0 if rope_prefix is None else rope_prefix.numel() * rope_prefix.element_size()
        dup_compressed = max(0, info['compressed_memory'] - residual) / 2
        dup_original = max(0, info['original_memory'] - residual) / 2
        info['compressed_memory'] = dup_compressed + residual + rope_prefix_bytes
        info['original_memory'] = dup_original + residual + rope_prefix_bytes
        info['dense_rope_memory'] = rope_prefix_bytes + residual_rope
        info['dense_rope_prefix_seq_len'] = self._dense_rope_prefix_seq_len
        info['rope_outlier_ratios'] = 0.0
        return info

    def release_dense_rope(self) -> None:
        self._res_v.clear()
        self._rope_prefix.clear()

    def release(self) -> None:
        super().release()
        self._rope_prefix.clear()


class MLAFloat11Cache(Float11Cache):
    """Lossless float11 cache for MLA latent + rope-key tensors
    (reference: mla_float_cache_utils.py:448-666)."""

    def __init__(
        self,
        config,
        right=None,
        exp_bits=None,
        latent_right: int = 127,
        rope_right: int = 127,
        latent_nbits: int = 4,
        rope_nbits: int = 4,
        need_adjust: bool = False,
        update_steps: int = 64,
        residual_length: int = 0,
        block_size: int = 128,
        layout: str = 'segmented_tiled',
        seq_tile_size: Optional[int] = None,
        mla_cache_mode: str = 'auto',
        validate_shapes: bool = True,
        compress_rope: bool = True,
        dense_workspace: str = 'shared',
        hist_reduce=None,
    ):
        text_config = config.get_text_config(decoder=True)
        self.mla_cache_mode = str(mla_cache_mode)
        self.validate_shapes = bool(validate_shapes)
        self.compress_rope = bool(compress_rope)
        self._shape_warning_emitted = False
        self.expected_latent_dim = getattr(text_config, 'kv_lora_rank', None)
        self.expected_rope_dim = getattr(text_config, 'qk_rope_head_dim', None)
        num_layers = int(text_config.num_hidden_layers)
        if (right is None) != (exp_bits is None):
            raise ValueError('MLAFloat11Cache expects right and exp_bits to be provided together.')
        if right is not None and exp_bits is not None:
            self.rights = _normalize_component_pairs(right, num_layers, 'right')
            self.nbits = _normalize_component_pairs(exp_bits, num_layers, 'exp_bits')
            latent_right, rope_right = int(self.rights[0][0]), int(self.rights[0][1])
            latent_nbits, rope_nbits = int(self.nbits[0][0]), int(self.nbits[0][1])
        else:
            self.rights, self.nbits = _component_pairs(num_layers, latent_right, rope_right, latent_nbits, rope_nbits)
        self.latent_right, self.rope_right = int(latent_right), int(rope_right)
        self.latent_nbits, self.rope_nbits = int(latent_nbits), int(rope_nbits)

        if self.compress_rope:
            super().__init__(config=config, right=self.rights, exp_bits=self.nbits, need_adjust=need_adjust,
                             update_steps=update_steps, residual_length=residual_length, block_size=block_size,
                             layout=layout, seq_tile_size=seq_tile_size, dense_workspace=dense_workspace,
                             hist_reduce=hist_reduce)
            return
        layers = [
            MLALatentFloat11DenseRopeLayer(
                latent_right=int(self.rights[i][0]), latent_nbits=int(self.nbits[i][0]),
                residual_length=residual_length, block_size=block_size, layout=layout,
                seq_tile_size=seq_tile_size, dense_workspace=dense_workspace)
            for i in range(num_layers)]
        for layer in layers:
            layer.hist_reduce = hist_reduce
        self._init_adjust_schedule(need_adjust, update_steps, block_size, layout)
        self.peak_mem = 0
        self.layout = layout
        self.seq_tile_size = seq_tile_size if seq_tile_size is not None else block_size
        self.auto_init_compress_params = False
        Cache.__init__(self, layers=layers)

    def _validate_update_shapes(self, first: torch.Tensor, second: torch.Tensor) -> None:
        """One warning at most, never an exception (reference: :550-595)."""
        if not self.validate_shapes or self._shape_warning_emitted:
            return
        msg = None
        if first.dim() != 4 or second.dim() != 4:
            msg = ('MLAFloat11Cache expects 4D cache tensors [batch, heads, seq, dim]. '
                   f'Got first={tuple(first.shape)}, second={tuple(second.shape)}.')
        elif first.shape[0] != second.shape[0] or first.shape[-2] != second.shape[-2]:
            msg = ('MLAFloat11Cache received cache tensors with different batch or sequence length: '
                   f'first={tuple(first.shape)}, second={tuple(second.shape)}.')
        elif self.mla_cache_mode == 'latent' and (first.shape[1] != 1 or second.shape[1] != 1):
            msg = ('MLAFloat11Cache latent mode normally receives [batch, 1, seq, dim] tensors '
                   f'for compressed_kv and k_pe. Got first={tuple(first.shape)}, second={tuple(second.shape)}.')
        elif self.mla_cache_mode in {'auto', 'latent'}:
            if self.expected_latent_dim is not None and int(first.shape[-1]) != int(self.expected_latent_dim):
                msg = ('MLAFloat11Cache first tensor last dim does not match config.kv_lora_rank: '
                       f'got {int(first.shape[-1])}, expected {int(self.expected_latent_dim)}. '
                       'If this model passes expanded full key/value tensors, use --mla_cache_mode expanded.')
            elif self.expected_rope_dim is not None and int(second.shape[-1]) != int(self.expected_rope_dim):
                msg = ('MLAFloat11Cache second tensor last dim does not match config.qk_rope_head_dim: '
                       f'got {int(second.shape[-1])}, expected {int(self.expected_rope_dim)}. '
                       'If this model passes expanded full key/value tensors, use --mla_cache_mode expanded.')
        if msg is not None:
            warnings.warn(msg, RuntimeWarning)
            self._shape_warning_emitted = True

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[dict] = None):
        """reference: :597-641."""
        self._validate_update_shapes(key_states, value_states)
        if self.compress_rope:
            return super().update(key_states, value_states, layer_idx, cache_kwargs)
        if self.layer_class_to_replicate is not None:
            while len(self.layers) <= layer_idx:
                self.layers.append(self.layer_class_to_replicate())
        layer = self.layers[layer_idx]
        if self._segmented_adjust and layer_idx in self._pending_adjusts and layer.has_pending_adjust_work():
            keys_params = self._take_pending(layer_idx)
            if layer.has_pending_adjust_recompress():
                layer.apply_pending_adjust_recompress_if_needed(keys_params, keys_params)
            else:
                layer.apply_pending_dense_block_if_needed(keys_params, keys_params)
        if self._segmented_adjust and layer.has_pending_dense_block() and not layer.has_pending_adjust_work():
            layer.apply_pending_dense_block_if_needed()
        need_adjust = self.need_adjust and self.steps % self.update_steps == 0
        result = layer.update(key_states, value_states, need_adjust, cache_kwargs)
        keys_exp_count = result['keys_exp_count']
        if need_adjust and keys_exp_count is not None:
            if layer_idx in self._pending_adjusts:
                self._take_pending(layer_idx)
            # the reference hands this to a thread pool and reads it at the layer's next update;
            # computed here, delivered at the same point
            if layer.hist_reduce is not None:
                keys_exp_count = layer.hist_reduce(keys_exp_count)
            try:
                self._pending_adjusts[layer_idx] = ('ok', codec.analysis_best_bits(codec.read_back(keys_exp_count.to(torch.int32))))
            except IndexError as exc:
                self._pending_adjusts[layer_idx] = ('err', exc)
        if layer_idx == len(self.layers) - 1:
            self.steps += 1
        return result['key_states'], result['value_states']

    def _take_pending(self, layer_idx: int):
        kind, payload = self._pending_adjusts.pop(layer_idx)
        if kind == 'err':
            raise payload
        return payload

    def get_memory(self) -> dict:
        """reference: :643-659."""
        info = super().get_memory()
        info.update(
            mla_cache_mode=self.mla_cache_mode, mla_compress_rope=self.compress_rope,
            mla_latent_right=self.latent_right, mla_rope_right=self.rope_right,
            mla_latent_nbits=self.latent_nbits, mla_rope_nbits=self.rope_nbits,
            mla_rights=self.rights, mla_nbits=self.nbits,
            mla_expected_latent_dim=self.expected_latent_dim, mla_expected_rope_dim=self.expected_rope_dim)
        info['latent_update_times'] = info.get('keys_update_times', 0)
        info['rope_update_times'] = info.get('values_update_times', 0)
        info['latent_outlier_ratios'] = info.get('keys_outlier_ratios', 0.0)
        info['rope_outlier_ratios'] = info.get('values_outlier_ratios', 0.0)
        return info

    def synchronize_and_release(self) -> None:
        super().synchronize_and_release()
        if not self.compress_rope:
            for layer in self.layers:
                if hasattr(layer, 'release_dense_rope'):
                    layer.release_dense_rope()

"""Update schedules used to pin the cache state machine.

A scenario fixes the cache constructor arguments and a deterministic sequence of
``update(k, v, layer)`` calls (seeded CPU tensors).  The same scenario is replayed through
the reference implementation (to write ``tests/golden/*.json``), through the host logic over
the CPU oracle (``-m "not gpu"``) and through the CUDA path (``-m gpu``).  What is compared is
a digest of the resulting cache: window and code length of every packed block, SHA-256 of its
four byte streams, the counters of ``get_memory()`` and the current parameters.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Callable, Iterator

import numpy as np
import torch

from tests import synth


@dataclass
class Scenario:
    name: str
    kind: str                      # 'float11' or 'mla'
    num_layers: int
    cache_kwargs: dict
    steps: Callable[[], Iterator]  # yields lists [(k, v) per layer] per forward pass
    config_extra: dict = field(default_factory=dict)


class StubConfig:
    """The only things the caches read from a model config."""

    def __init__(self, num_hidden_layers: int, **extra):
        self.num_hidden_layers = num_hidden_layers
        for k, v in extra.items():
            setattr(self, k, v)

    def get_text_config(self, decoder: bool = True):
        return self


def _kv_stream(shape_k, shape_v, seed, prefill, decode, scale_after=None, scale=1.0, layers=1, chunk=1):
    """prefill tokens in one update, then `decode` tokens `chunk` at a time; values are scaled
    by `scale` from token index `scale_after` on (forces the adjuster to move the window)."""
    def gen():
        B, H, Dk = shape_k
        _, Hv, Dv = shape_v
        total = prefill + decode
        ks = [synth.kv_tensor((B, H, total, Dk), seed=seed + 10 * l, mu=-0.3 + 0.4 * l, key_offset=True) for l in range(layers)]
        vs = [synth.kv_tensor((B, Hv, total, Dv), seed=seed + 10 * l + 5, mu=0.2 - 0.3 * l) for l in range(layers)]
        if scale_after is not None:
            for t in ks + vs:
                t[:, :, scale_after:] = (t[:, :, scale_after:].float() * scale).to(torch.bfloat16)
        pos = 0
        if prefill:
            yield [(ks[l][:, :, :prefill], vs[l][:, :, :prefill]) for l in range(layers)]
            pos = prefill
        while pos < total:
            n = min(chunk, total - pos)
            yield [(ks[l][:, :, pos:pos + n], vs[l][:, :, pos:pos + n]) for l in range(layers)]
            pos += n
    return gen


def _adj(**kw):
    base = dict(need_adjust=True, update_steps=128, residual_length=0, block_size=128, layout='segmented_tiled')
    base.update(kw)
    return base


SCENARIOS = {s.name: s for s in [
    # single-layer round trip: one 2048-token update of K,V [1, 8, 2048, 128]
    Scenario('config0_prefill_2048', 'float11', 1,
             dict(right=[(130, 129)], exp_bits=[(3, 3)], **_adj()),
             _kv_stream((1, 8, 128), (1, 8, 128), seed=0, prefill=2048, decode=0)),
    # ragged prefill, then decode past two block boundaries; two layers with different windows
    Scenario('prefill300_decode299', 'float11', 2,
             dict(right=[(129, 128), (131, 127)], exp_bits=[(3, 3), (4, 3)], **_adj()),
             _kv_stream((1, 4, 64), (1, 4, 64), seed=3, prefill=300, decode=299, layers=2)),
    # prefill a whole number of blocks, then single tokens whose scale jumps x64 at token 356:
    # blocks are staged exactly on adjust steps, the window follows the data
    Scenario('scale_shift_adjust', 'float11', 1,
             dict(right=[(128, 128)], exp_bits=[(3, 3)], **_adj()),
             _kv_stream((1, 2, 64), (1, 2, 64), seed=7, prefill=256, decode=520, scale_after=356, scale=64.0)),
    # adjuster off: blocks filled during decode stay dense for good
    Scenario('no_adjust', 'float11', 1,
             dict(right=129, exp_bits=3, need_adjust=False, update_steps=64, block_size=128, layout='segmented_tiled'),
             _kv_stream((1, 2, 32), (1, 2, 32), seed=11, prefill=200, decode=200)),
    # batch 2, prefill of exactly two blocks, 260 decode tokens
    Scenario('batch2_aligned', 'float11', 1,
             dict(right=[(129, 129)], exp_bits=[(3, 3)], **_adj()),
             _kv_stream((2, 2, 32), (2, 2, 32), seed=13, prefill=256, decode=260)),
    # no prefill at all: 300 single-token updates
    Scenario('decode_only', 'float11', 1,
             dict(right=[(129, 129)], exp_bits=[(3, 3)], **_adj()),
             _kv_stream((1, 2, 32), (1, 2, 32), seed=17, prefill=0, decode=300)),
    # update_steps is rounded up to a block multiple (100 -> 128); multi-token appends
    Scenario('chunked_appends', 'float11', 1,
             dict(right=[(129, 129)], exp_bits=[(3, 3)], **_adj(update_steps=100)),
             _kv_stream((1, 2, 32), (1, 2, 32), seed=19, prefill=130, decode=420, chunk=7)),
    # window (-4, 3]: every element escapes (the reference's own validation fixture uses right=3)
    Scenario('all_escape', 'float11', 1,
             dict(right=3, exp_bits=3, need_adjust=False, update_steps=0, block_size=128, layout='segmented_tiled'),
             _kv_stream((1, 2, 16), (1, 2, 16), seed=2026, prefill=128, decode=3)),
    # MLA latent cache, rope key compressed as the "values" tensor
    Scenario('mla_compress_rope', 'mla', 2,
             dict(right=[(128, 127), (129, 127)], exp_bits=[(3, 4), (3, 4)], compress_rope=True, **_adj()),
             _kv_stream((2, 1, 64), (2, 1, 16), seed=23, prefill=200, decode=200, layers=2),
             config_extra=dict(kv_lora_rank=64, qk_rope_head_dim=16)),
    # flat ('legacy') layout: every full block is packed at once, also in decode; windows proposed on
    # an adjust step are adopted at the next one (period 64 is NOT rounded for this layout)
    Scenario('legacy_layout_adjust', 'float11', 1,
             dict(right=[(128, 128)], exp_bits=[(3, 3)], need_adjust=True, update_steps=64, residual_length=0,
                  block_size=128, layout='legacy'),
             _kv_stream((1, 2, 32), (1, 2, 32), seed=31, prefill=200, decode=330, scale_after=260, scale=64.0)),
    # unified 'tiled' layout without the adjuster: one state per tensor, planes in [b][h][tile] order
    Scenario('tiled_layout_fixed', 'float11', 1,
             dict(right=[(129, 128)], exp_bits=[(3, 4)], need_adjust=False, update_steps=0, residual_length=0,
                  block_size=128, layout='tiled'),
             _kv_stream((2, 2, 32), (2, 2, 32), seed=37, prefill=300, decode=260)),
    # MLA with the rope key kept dense
    Scenario('mla_dense_rope', 'mla', 1,
             dict(right=[(128, 127)], exp_bits=[(3, 4)], compress_rope=False, **_adj()),
             _kv_stream((2, 1, 64), (2, 1, 16), seed=29, prefill=200, decode=330, scale_after=300, scale=32.0),
             config_extra=dict(kv_lora_rank=64, qk_rope_head_dim=16)),
]}


def _sha(t) -> str:
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu().contiguous()
        a = t.view(torch.uint8).numpy() if t.numel() else np.zeros(0, np.uint8)
    else:
        a = np.ascontiguousarray(t).view(np.uint8)
    return hashlib.sha256(a.tobytes()).hexdigest()[:24]


def segment_digest(state: dict) -> dict:
    """Digest of one exported segment state (works for the reference's dicts and ours)."""
    return {
        'right': int(state['right']), 'nbits': int(state['nbits']), 'left': int(state['left']),
        'shape': [int(v) for v in state['original_shape']],
        'n_escapes': int(state['invalid_exp'].numel()),
        'sign_mass_data': _sha(state['sign_mass_data']), 'exp_data': _sha(state['exp_data']),
        'invalid_exp': _sha(state['invalid_exp']), 'tile_invalid_base': _sha(state['tile_invalid_base'].to(torch.int32)),
    }


_MEMORY_KEYS = (
    'compressed_memory', 'original_memory', 'keys_outlier_ratios', 'values_outlier_ratios', 'keys_update_times',
    'values_update_times', 'keys_update_proposals', 'values_update_proposals', 'materialize_calls',
    'materialize_cache_hits', 'stored_compressed_prefix_seq_len', 'stored_residual_seq_len',
    'compressed_block_flushes', 'compressed_tokens_flushed', 'residual_tokens_kept',
    'stored_compressed_block_count', 'prefill_reuse_hits', 'adjust_recompresses', 'delayed_adjust_block_flushes',
)


def _n_packed_blocks(layer) -> int:
    layout = getattr(layer, 'layout', 'segmented_tiled')
    if layout == 'legacy':
        return len(layer._compressed_prefix_key_blocks)
    if layout == 'tiled':
        st = layer._compressed_prefix_key_state
        return 0 if st is None else int(st['num_sequence_tiles'])
    return len(layer._compressed_prefix_key_segments)


def legacy_block_digest(state: dict) -> dict:
    """Digest of one flat ('legacy') block state (``CompressorBitMap.export_state``)."""
    return {
        'right': int(state['right']), 'nbits': int(state['nbits']), 'left': int(state['left']),
        'shape': [int(v) for v in state['original_shape']], 'n_escapes': int(state['invalid_exp'].numel()),
        'sign_mass_data': _sha(state['sign_mass_data']), 'exp_data': _sha(state['exp_data']),
        'invalid_exp': _sha(state['invalid_exp']), 'block_base': _sha(state['block_base'].to(torch.int64)),
    }


def layer_digest(layer) -> dict:
    mem = layer.get_memory()
    layout = getattr(layer, 'layout', 'segmented_tiled')
    if layout == 'legacy':
        key_part = [legacy_block_digest(s) for s in layer._compressed_prefix_key_blocks]
        value_part = [legacy_block_digest(s) for s in layer._compressed_prefix_value_blocks]
    elif layout == 'tiled':
        ks, vs = layer._compressed_prefix_key_state, layer._compressed_prefix_value_state
        key_part = [] if ks is None else [segment_digest(ks)]
        value_part = [] if vs is None else [segment_digest(vs)]
    else:
        key_part = [segment_digest(s) for s in layer._compressed_prefix_key_segments]
        value_part = [segment_digest(s) for s in layer._compressed_prefix_value_segments]
    out = {
        'key_segments': key_part,
        'value_segments': value_part,
        'memory': {k: mem[k] for k in _MEMORY_KEYS},
        'params': [int(layer.keys_right), int(layer.keys_nbits), int(layer.values_right), int(layer.values_nbits)],
        'new_params': [int(layer.new_keys_right), int(layer.new_keys_nbits), int(layer.new_values_right),
                       int(layer.new_values_nbits)],
        'seq_length': int(layer.get_seq_length()),
    }
    for extra in ('dense_rope_memory', 'dense_rope_prefix_seq_len'):
        if extra in mem:
            out['memory'][extra] = mem[extra]
    return out


def run_scenario(sc: Scenario, make_cache, device='cpu', check_dense: bool = True, trace_every: int = 0):
    """Replay a scenario.  ``make_cache(kind, config, **kwargs)`` builds the cache under test.
    Every update's returned dense K/V is compared, bit for bit, with the concatenation of the
    inputs so far.  Returns the digest (final state plus optional intermediate snapshots)."""
    cfg = StubConfig(sc.num_layers, **sc.config_extra)
    cache = make_cache(sc.kind, cfg, **sc.cache_kwargs)
    seen_k = [[] for _ in range(sc.num_layers)]
    seen_v = [[] for _ in range(sc.num_layers)]
    snapshots = []
    for step, per_layer in enumerate(sc.steps()):
        for l, (k, v) in enumerate(per_layer):
            kd, vd = k.to(device), v.to(device)
            out_k, out_v = cache.update(kd, vd, l)
            seen_k[l].append(k)
            seen_v[l].append(v)
            if check_dense:
                exp_k = torch.cat(seen_k[l], dim=-2)
                exp_v = torch.cat(seen_v[l], dim=-2)
                assert out_k.shape == exp_k.shape, (step, l, out_k.shape, exp_k.shape)
                assert torch.equal(out_k.cpu().view(torch.int16), exp_k.view(torch.int16)), f'keys differ at step {step} layer {l}'
                assert torch.equal(out_v.cpu().view(torch.int16), exp_v.view(torch.int16)), f'values differ at step {step} layer {l}'
        if trace_every and (step % trace_every == 0):
            snapshots.append({'step': step, 'layers': [
                {'params': [int(x.keys_right), int(x.keys_nbits), int(x.values_right), int(x.values_nbits)],
                 'n_segments': _n_packed_blocks(x)} for x in cache.layers]})
    digest = {'layers': [layer_digest(x) for x in cache.layers], 'snapshots': snapshots,
              'steps': int(cache.steps), 'update_steps': int(cache.update_steps)}
    for l in range(sc.num_layers if check_dense else 0):
        mk, mv = cache.materialize_layer(l)
        assert torch.equal(mk.cpu().view(torch.int16), torch.cat(seen_k[l], dim=-2).view(torch.int16))
        assert torch.equal(mv.cpu().view(torch.int16), torch.cat(seen_v[l], dim=-2).view(torch.int16))
    return digest, cache


def stress_scenario(batch=4, heads=8, dim=128, prefill=512, decode=384, layers=2, seed=41):
    """Reduced replica of the multi-GPU stress configuration: after `prefill` tokens the scale of
    half the heads doubles, 0.1 % of the values carry exponents outside the calibrated window and
    0.01 % are zero/subnormal; the prompt is a whole number of blocks and the rest arrives one
    token at a time, so blocks fill exactly on adjust steps."""
    def gen():
        total = prefill + decode
        ks, vs = [], []
        for l in range(layers):
            k = synth.kv_tensor((batch, heads, total, dim), seed=seed + 7 * l, key_offset=True)
            v = synth.kv_tensor((batch, heads, total, dim), seed=seed + 7 * l + 3)
            for t in (k, v):
                t[:, heads // 2:, prefill:] = (t[:, heads // 2:, prefill:].float() * 2.0).to(torch.bfloat16)
            ks.append(synth.inject_escapes(k, seed + 100 + l, left=122, right=129))
            vs.append(synth.inject_escapes(v, seed + 200 + l, left=121, right=128))
        yield [(ks[l][:, :, :prefill], vs[l][:, :, :prefill]) for l in range(layers)]
        for pos in range(prefill, total):
            yield [(ks[l][:, :, pos:pos + 1], vs[l][:, :, pos:pos + 1]) for l in range(layers)]
    return Scenario('stress_replica', 'float11', layers,
                    dict(right=[(129, 128)] * layers, exp_bits=[(3, 3)] * layers, **_adj()), gen)

"""Host logic of Float11Cache / MLAFloat11Cache replayed on the CPU over the oracle codec and
compared with the digests the reference implementation produced for the same scenarios
(tests/golden/state_machine.json): per-block window, code length and SHA-256 of the four byte
streams, every counter of get_memory(), current and proposed parameters.  The dense K/V
returned by every update are compared bit for bit with the inputs inside run_scenario."""
import json
import os
import warnings

import pytest

from tests import oracle_codec, scenarios

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), 'golden', 'state_machine.json')))


def make_cache_factory(dense_workspace='shared'):
    from adacode_b200.float_cache_utils import Float11Cache
    from adacode_b200.mla_float_cache_utils import MLAFloat11Cache

    def make(kind, cfg, **kw):
        kw = dict(kw, dense_workspace=dense_workspace)
        return MLAFloat11Cache(cfg, **kw) if kind == 'mla' else Float11Cache(cfg, **kw)
    return make


def assert_digest_equal(got, exp, where=''):
    assert got['steps'] == exp['steps'] and got['update_steps'] == exp['update_steps']
    assert got['snapshots'] == exp['snapshots'], f'{where}: parameter/segment trace differs'
    for l, (g, e) in enumerate(zip(got['layers'], exp['layers'])):
        assert g['params'] == e['params'], f'{where} layer {l}: params {g["params"]} != {e["params"]}'
        assert g['new_params'] == e['new_params'], f'{where} layer {l}: proposals differ'
        assert g['seq_length'] == e['seq_length']
        for side in ('key_segments', 'value_segments'):
            assert len(g[side]) == len(e[side]), f'{where} layer {l}: {side} count'
            for j, (gs, es) in enumerate(zip(g[side], e[side])):
                assert gs == es, f'{where} layer {l} {side}[{j}]: {gs} != {es}'
        for k, ev in e['memory'].items():
            gv = g['memory'][k]
            if isinstance(ev, float):
                assert gv == pytest.approx(ev, rel=1e-12, abs=1e-15), f'{where} layer {l}: memory[{k}]'
            else:
                assert gv == ev, f'{where} layer {l}: memory[{k}] {gv} != {ev}'


@pytest.fixture
def cpu_codec(monkeypatch):
    import adacode_b200.float_cache_utils as fc
    import adacode_b200.mla_float_cache_utils as mc
    monkeypatch.setattr(fc, 'codec', oracle_codec)
    monkeypatch.setattr(mc, 'codec', oracle_codec)


@pytest.mark.parametrize('name', sorted(scenarios.SCENARIOS))
@pytest.mark.parametrize('dense_workspace', ['shared', 'layer'])
def test_scenario_matches_reference(cpu_codec, name, dense_workspace):
    if dense_workspace == 'layer' and name not in ('prefill300_decode299', 'scale_shift_adjust', 'mla_dense_rope'):
        pytest.skip('per-layer mirror covered on three scenarios')
    with warnings.catch_warnings():
        warnings.simplefilter('ignore')
        digest, _ = scenarios.run_scenario(scenarios.SCENARIOS[name], make_cache_factory(dense_workspace), trace_every=16)
    assert_digest_equal(digest, GOLDEN[name], name)


@pytest.mark.parametrize('name', ['prefill300_decode299', 'scale_shift_adjust'])
def test_fused_decode_mode_keeps_the_packing_schedule(cpu_codec, name):
    """Inside ``hf_attention.fused_decode`` single-token updates skip the dense rebuild and hand
    back the new token only; the cache must still end in the reference's state: same windows,
    same bytes of every packed block, same adjuster counters (only the materialise counters
    differ, by construction)."""
    from adacode_b200 import hf_attention
    made = []

    def make(kind, cfg, **kw):
        cache = make_cache_factory('shared')(kind, cfg, **kw)
        made.append(cache)
        return cache

    class Fused:
        """run_scenario builds the cache itself: switch fused mode on right after construction."""
        def __call__(self, kind, cfg, **kw):
            cache = make(kind, cfg, **kw)
            self.ctx = hf_attention.fused_decode(cache)
            self.ctx.__enter__()
            return cache

    factory = Fused()
    sc = scenarios.SCENARIOS[name]
    seen = {'single': 0}
    try:
        with warnings.catch_warnings():
            warnings.simplefilter('ignore')
            cfg = scenarios.StubConfig(sc.num_layers, **sc.config_extra)
            cache = factory(sc.kind, cfg, **sc.cache_kwargs)
            for per_layer in sc.steps():
                for l, (k, v) in enumerate(per_layer):
                    out_k, out_v = cache.update(k, v, l)
                    if k.shape[-2] == 1 and cache.layers[l].get_seq_length() > 1:
                        assert out_k.shape == k.shape and out_v.shape == v.shape     # the new token, not the cache
                        seen['single'] += 1
    finally:
        factory.ctx.__exit__(None, None, None)
    assert seen['single'] > 0 and not cache._fused_decode
    exp = GOLDEN[name]
    got = {'layers': [scenarios.layer_digest(x) for x in cache.layers]}
    for l, (g, e) in enumerate(zip(got['layers'], exp['layers'])):
        assert g['params'] == e['params'] and g['new_params'] == e['new_params'] and g['seq_length'] == e['seq_length']
        assert g['key_segments'] == e['key_segments'] and g['value_segments'] == e['value_segments']
        for k, ev in e['memory'].items():
            if k.startswith('materialize'):
                continue
            gv = g['memory'][k]
            assert (gv == pytest.approx(ev, rel=1e-12, abs=1e-15)) if isinstance(ev, float) else gv == ev, (l, k)
    assert int(cache.steps) == exp['steps']

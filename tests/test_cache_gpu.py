"""GPU parity of the cache classes: every scenario replayed through the CUDA kernels must end
in the digest the reference produced (window, code length and SHA-256 of every packed block's
byte streams, all counters), and every update must return K/V bit-identical to the inputs."""
import io
import json
import os
import pickle
import warnings

import numpy as np
import pytest
import torch

from tests import scenarios, synth
from tests.test_state_machine_cpu import GOLDEN, assert_digest_equal, make_cache_factory

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('name', sorted(scenarios.SCENARIOS))
def test_scenario_on_gpu_matches_reference(cuda_device, name):
    with warnings.catch_warnings():
        warnings.simplefilter('ignore')
        digest, cache = scenarios.run_scenario(scenarios.SCENARIOS[name], make_cache_factory('shared'),
                                               device=cuda_device, trace_every=16)
    assert_digest_equal(digest, GOLDEN[name], name)
    from adacode_b200 import codec
    codec.check_device_status(cuda_device)


@pytest.mark.parametrize('name', ['prefill300_decode299', 'mla_dense_rope'])
def test_per_layer_mirror_on_gpu(cuda_device, name):
    with warnings.catch_warnings():
        warnings.simplefilter('ignore')
        digest, _ = scenarios.run_scenario(scenarios.SCENARIOS[name], make_cache_factory('layer'),
                                           device=cuda_device, trace_every=16)
    assert_digest_equal(digest, GOLDEN[name], name)


def test_strided_projection_input_and_cache_view(cuda_device):
    """Keys arrive as a [B, S, H, D] projection viewed [B, H, S, D]; no host-side copy is needed."""
    from adacode_b200 import Float11Cache
    from tests import synth
    cfg = scenarios.StubConfig(1)
    cache = Float11Cache(cfg, right=[(129, 129)], exp_bits=[(3, 3)], need_adjust=True, update_steps=128,
                         block_size=128, layout='segmented_tiled')
    base_k = synth.kv_tensor((2, 300, 4, 64), seed=1, key_offset=True).to(cuda_device)
    base_v = synth.kv_tensor((2, 300, 4, 64), seed=2).to(cuda_device)
    k, v = base_k.transpose(1, 2), base_v.transpose(1, 2)
    out_k, out_v = cache.update(k, v, 0)
    assert out_k is k and out_v is v                      # prefill hands the inputs back
    assert cache.get_seq_length(0) == 300
    mk, mv = cache.materialize_layer(0)
    assert mk.is_contiguous() and torch.equal(mk, k) and torch.equal(mv, v)
    view = cache.get_layer_cache_view(0)
    assert view['decode_impl'] == 'materialize_dense' and view['compressed_prefix_seq_len'] == 256
    assert view['compressed_prefix_key']['num_segments'] == 2 and view['residual_keys'].shape[-2] == 44
    assert view['seq_length'] == 300
    mem = cache.get_memory()
    assert 0 < mem['kv_compressed_memory'] < mem['kv_original_memory']
    params = cache.get_compress_params()
    assert params['kv_current_rights'] == [(129, 129)] and params['kv_current_nbits'] == [(3, 3)]
    cache.synchronize_and_release()
    assert cache.layers[0].get_memory()['compressed_memory'] == 0


def test_pickle_round_trip(cuda_device):
    from adacode_b200 import Float11Cache
    from tests import synth
    cfg = scenarios.StubConfig(1)
    cache = Float11Cache(cfg, right=129, exp_bits=3, need_adjust=True, update_steps=128, block_size=128,
                         layout='segmented_tiled')
    k = synth.kv_tensor((1, 2, 200, 32), seed=4).to(cuda_device)
    v = synth.kv_tensor((1, 2, 200, 32), seed=5).to(cuda_device)
    cache.update(k, v, 0)
    cache.update(k[:, :, :1], v[:, :, :1], 0)
    clone = pickle.loads(pickle.dumps(cache))
    a, b = cache.materialize_layer(0)
    a, b = a.clone(), b.clone()
    c, d = clone.materialize_layer(0)
    assert torch.equal(a, c) and torch.equal(b, d)
    assert clone.layers[0].segment_params() == cache.layers[0].segment_params()


def test_hf_generate_matches_dynamic_cache(cuda_device):
    """A small random-init Llama generates the same token ids with Float11Cache as with
    DynamicCache: the K/V attention sees are bit-identical, so the logits are too."""
    from transformers import DynamicCache, LlamaConfig, LlamaForCausalLM
    from adacode_b200 import Float11Cache
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=8,
                      num_key_value_heads=2, head_dim=32, vocab_size=1000, max_position_embeddings=1024)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).to(cuda_device).eval()
    ids = torch.randint(0, 1000, (2, 200), device=cuda_device)
    kw = dict(max_new_tokens=140, min_new_tokens=140, do_sample=False, pad_token_id=0)
    with torch.no_grad():
        ref = model.generate(ids, past_key_values=DynamicCache(config=cfg), **kw)
        cache = Float11Cache(cfg, right=129, exp_bits=4, need_adjust=True, update_steps=128, block_size=128,
                             layout='segmented_tiled')
        out = model.generate(ids, past_key_values=cache, **kw)
    assert torch.equal(ref, out)
    mem = cache.get_memory()
    assert mem['compressed_block_flushes'] >= 2 * 2 and mem['kv_compressed_memory'] < mem['kv_original_memory']


def _oracle_factory():
    """The same host classes over the CPU oracle codec (the state machine itself is pinned to the
    reference by tests/golden/state_machine.json)."""
    import adacode_b200.float_cache_utils as fc
    import adacode_b200.mla_float_cache_utils as mc
    from tests import oracle_codec
    real = (fc.codec, mc.codec)

    class Swap:
        def __enter__(self):
            fc.codec = mc.codec = oracle_codec

        def __exit__(self, *exc):
            fc.codec, mc.codec = real
    return Swap()


def test_stress_replica_gpu_equals_cpu_oracle(cuda_device):
    """Reduced replica of the stress configuration (scale shift for half the heads, injected
    out-of-window and zero exponents, single-token appends): the CUDA cache ends in exactly the
    state the oracle-backed host logic ends in — every block's window, bytes and all counters."""
    sc = scenarios.stress_scenario(batch=2, heads=4, dim=128, prefill=256, decode=300, layers=2)
    with warnings.catch_warnings():
        warnings.simplefilter('ignore')
        gpu_digest, _ = scenarios.run_scenario(sc, make_cache_factory('shared'), device=cuda_device, trace_every=32)
        with _oracle_factory():
            cpu_digest, _ = scenarios.run_scenario(sc, make_cache_factory('shared'), device='cpu', trace_every=32)
    assert_digest_equal(gpu_digest, cpu_digest, 'stress_replica')
    changed = sum(l['memory']['keys_update_times'] + l['memory']['values_update_times'] for l in cpu_digest['layers'])
    assert changed > 0, 'the schedule is meant to make the adjuster move a window'
    assert all(l['key_segments'][0]['n_escapes'] > 0 for l in cpu_digest['layers'])


def test_mla_true_dimensions(cuda_device):
    """DeepSeek-V2-Lite shaped tensors: 512-dim latent, 64-dim rope key, both cache modes."""
    import numpy as np
    from adacode_b200 import MLAFloat11Cache
    from oracle import float11_oracle as O
    from tests import synth
    cfg = scenarios.StubConfig(1, kv_lora_rank=512, qk_rope_head_dim=64)
    lat = synth.kv_tensor((2, 1, 300, 512), seed=51, mu=-0.5, s=0.8)
    rope = synth.kv_tensor((2, 1, 300, 64), seed=52)
    for compress_rope in (True, False):
        cache = MLAFloat11Cache(cfg, right=[(128, 129)], exp_bits=[(3, 4)], need_adjust=True, update_steps=128,
                                block_size=128, compress_rope=compress_rope)
        with warnings.catch_warnings():
            warnings.simplefilter('error')           # dims match the config: no shape warning expected
            cache.update(lat[:, :, :260].to(cuda_device), rope[:, :, :260].to(cuda_device), 0)
        for t in range(260, 300):
            a, b = cache.update(lat[:, :, t:t + 1].to(cuda_device), rope[:, :, t:t + 1].to(cuda_device), 0)
        assert torch.equal(a.cpu().view(torch.int16), lat.view(torch.int16))
        assert torch.equal(b.cpu().view(torch.int16), rope.view(torch.int16))
        layer = cache.layers[0]
        seg = layer._key_segments[0]
        ref = O.pack_block(lat[:, :, :128].contiguous(), seg.right, seg.nbits)
        assert np.array_equal(seg.exp_data.cpu().numpy(), ref.exp_data)
        assert np.array_equal(seg.invalid_exp.cpu().numpy(), ref.invalid_exp)
        mem = cache.get_memory()
        assert mem['mla_compress_rope'] == compress_rope and mem['kv_compressed_memory'] < mem['kv_original_memory']


def test_calibration_producer_feeds_the_consumer(cuda_device, tmp_path):
    """``extract_exp_freq`` over a live ``DynamicCache`` gives the oracle's exponent histograms
    (prefill / decode split), two batches merge bin by bin, and the JSON it is written to yields
    the windows the calibration rule picks on those histograms."""
    import json
    from transformers import DynamicCache
    from adacode_b200 import export_initial_compress_parameters
    from adacode_b200.export_kvcache_status import extract_exp_freq, merge_exp_freq
    from oracle import float11_oracle as O
    layers, prefill = 3, 200
    results, tensors = [], []
    for batch in range(2):
        cache = DynamicCache()
        per_layer = []
        for l in range(layers):
            k = synth.kv_tensor((2, 4, 260, 64), seed=100 + 10 * batch + l, key_offset=True)
            v = synth.kv_tensor((2, 4, 260, 64), seed=200 + 10 * batch + l)
            cache.update(k.to(cuda_device), v.to(cuda_device), l)
            per_layer.append((k, v))
        tensors.append(per_layer)
        results.append(extract_exp_freq(cache, 'exp', prefill_len=prefill))
    for batch in range(2):
        for l in range(layers):
            k, v = tensors[batch][l]
            got = results[batch][l]
            assert got['prefill_keys'] == O.exponent_hist(k[:, :, :prefill].contiguous()).tolist()
            assert got['decode_keys'] == O.exponent_hist(k[:, :, prefill:].contiguous()).tolist()
            assert got['prefill_values'] == O.exponent_hist(v[:, :, :prefill].contiguous()).tolist()
            assert got['decode_values'] == O.exponent_hist(v[:, :, prefill:].contiguous()).tolist()
    merged = merge_exp_freq(results[0], results[1])
    assert merged[1]['decode_keys'] == [a + b for a, b in zip(results[0][1]['decode_keys'], results[1][1]['decode_keys'])]
    path = tmp_path / 'stats.json'
    path.write_text(json.dumps({'c4': {str(l): merged[l] for l in range(layers)}}))
    rights, nbits = export_initial_compress_parameters(str(path), 'c4', 'merge')
    for l in range(layers):
        kh = np.asarray(merged[l]['prefill_keys']) + np.asarray(merged[l]['decode_keys'])
        vh = np.asarray(merged[l]['prefill_values']) + np.asarray(merged[l]['decode_values'])
        assert (rights[l][0], nbits[l][0]) == tuple(O.calibrate_coo(kh))
        assert (rights[l][1], nbits[l][1]) == tuple(O.calibrate_coo(vh))
    whole = extract_exp_freq(cache)                      # no split
    assert whole[0]['keys'] == O.exponent_hist(tensors[1][0][0]).tolist()


def test_runner_writes_reference_shaped_records(cuda_device, tmp_path, monkeypatch):
    """``main_lossless_comp`` with ``--use_synthetic_data --random_init``: the calibration JSON is
    produced on the spot, the float11 run generates the token ids of the DynamicCache run, and the
    per-batch record carries the reference's keys (main_lossless_comp.py:342-458)."""
    import json
    from adacode_b200 import main_lossless_comp as runner
    monkeypatch.chdir(tmp_path)
    common = ['--model_config_name', 'llama_3p1_8B_config', '--use_synthetic_data', '--synthetic_seq_length', '300',
              '--batch_size', '2', '--num_seqence', '2', '--max_new_tokens', '140', '--min_new_tokens', '140',
              '--random_init', '--random_init_layers', '2']
    recs = {}
    for impl, extra in (('dynamic', []), ('float11', ['--float11_need_adjust', '--float11_update_steps', '128'])):
        args = runner.get_parse().parse_args(common + ['--kv_cache_impl', impl, '--output_path', f'{impl}.json'] + extra)
        out = runner.run(args)
        on_disk = json.loads((tmp_path / f'{impl}.json').read_text())
        assert on_disk == out and len(out['synthetic']) == 1
        recs[impl] = out['synthetic'][0]
    assert (tmp_path / 'model_configs' / 'kv_test_Meta-Llama-3.1-8B-Instruct_exp.json').exists()
    f11, dyn = recs['float11'], recs['dynamic']
    assert f11['generated_output_head_32'] == dyn['generated_output_head_32']
    for key in ('dataset', 'sample_start_idx', 'batch_size', 'cache_mode', 'input_shape', 'total_input_tokens',
                'generate_time', 'total_new_tokens', 'tokens_per_second', 'kv_compressed_memory', 'kv_original_memory',
                'float11_layout', 'float11_need_adjust', 'float11_update_steps', 'cuda_peak_allocated_gib'):
        assert key in f11, key
    assert f11['input_shape'] == [2, 300] and f11['total_new_tokens'] == 2 * 140
    assert 0.6 < f11['kv_compressed_memory'] / f11['kv_original_memory'] < 1.0
    with pytest.raises(NotImplementedError):
        runner.run(runner.get_parse().parse_args(common + ['--kv_cache_impl', 'nvcomp_ans']))


def test_long_prefill_is_packed_in_several_launches(cuda_device, monkeypatch):
    """A prefill whose keys and values together would exceed the per-launch element limit is packed
    block range by block range; the cache ends in exactly the state of a single launch."""
    import adacode_b200.float_cache_utils as fc
    from adacode_b200 import Float11Cache
    k = synth.kv_tensor((2, 2, 128 * 7 + 30, 64), seed=71, key_offset=True).to(cuda_device)
    v = synth.kv_tensor((2, 2, 128 * 7 + 30, 64), seed=72).to(cuda_device)
    kw = dict(right=[(129, 128)], exp_bits=[(3, 3)], need_adjust=True, update_steps=128, block_size=128,
              layout='segmented_tiled')
    digests = []
    for limit in (2 ** 31 - 1, 2 * 3 * (2 * 2 * 128 * 64)):            # the second: three blocks per launch
        monkeypatch.setattr(fc, '_MAX_LAUNCH_ELEMS', limit)
        cache = Float11Cache(scenarios.StubConfig(1), **kw)
        cache.update(k, v, 0)
        dk, dv = cache.update(k[:, :, :1], v[:, :, :1], 0)               # applies the prefill's adjust proposal
        assert torch.equal(dk[:, :, :-1], k) and torch.equal(dv[:, :, :-1], v)
        digests.append(scenarios.layer_digest(cache.layers[0]))
    assert digests[0] == digests[1] and len(digests[0]['key_segments']) == 7

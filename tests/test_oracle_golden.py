"""CPU checks: the oracle against the byte-stream digests and adjuster results recorded from
the reference implementation, the host-side adjuster/calibration of the C library against the
same records, and that the built library exports every symbol its header declares."""
import ctypes
import json
import os
import re

import numpy as np
import pytest
import torch

from oracle import float11_oracle as O
from tests import scenarios, synth

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CODEC = json.load(open(os.path.join(HERE, 'golden', 'codec_vectors.json')))
ADJ = json.load(open(os.path.join(HERE, 'golden', 'adjuster_vectors.json')))


@pytest.mark.parametrize('case', CODEC['cases'], ids=lambda c: f"{c['path']}-s{c['seed']}-n{c['nbits']}")
def test_oracle_pack_matches_reference_digests(case):
    key_offset = case['path'] == 'pure_torch'
    x = synth.kv_tensor(tuple(case['shape']), seed=case['seed'], key_offset=key_offset)
    p = O.pack_block(x, case['right'], case['nbits'], need_hist=True)
    assert p.invalid_exp.size == case['n_escapes']
    assert scenarios._sha(p.sign_mass_data) == case['sign_mass_data']
    assert scenarios._sha(p.exp_data) == case['exp_data']
    assert scenarios._sha(p.invalid_exp) == case['invalid_exp']
    assert scenarios._sha(p.tile_invalid_base) == case['tile_invalid_base']
    assert p.left == case['left'] and p.compressed_bytes() == case['compressed_memory']
    assert [int(v) for v in p.hist] == case['hist']
    assert np.array_equal(O.unpack_block(p), O.as_u16(x))


def test_known_answers():
    torch.manual_seed(0)
    x = (torch.randn(1, 8, 128, 128) * 0.7).to(torch.bfloat16)
    x.view(-1)[5] = 0.0
    p = O.pack_block(x, 127, 3)
    ka = CODEC['known_answers']['randn07_right127_nbits3']
    assert p.invalid_exp.size == ka['n_escapes'] == 2980 and p.exp_data.size == ka['exp_bytes'] == 49152
    # the reference's validation fixture: window (-4, 3], every element escapes
    torch.manual_seed(2026)
    torch.randn(1, 2, 1, 16)
    k = torch.randn(1, 2, 128, 16).to(torch.bfloat16)
    v = torch.randn(1, 2, 128, 16).to(torch.bfloat16)
    fx = CODEC['known_answers']['validation_fixture_seed2026_right3']
    pk, pv = O.pack_block(k, 3, 3), O.pack_block(v, 3, 3)
    # that fixture ran the legacy layout, which stores one int64 base (torch.cumsum promotes) per 1024 elements
    legacy_bytes = sum(q.sign_mass_data.size + q.exp_data.size + q.invalid_exp.size + 8 * (k.numel() // 1024) for q in (pk, pv))
    assert legacy_bytes == fx['compressed_memory'] == 19520 and fx['original_memory'] == 16384
    assert pk.invalid_exp.size / k.numel() == fx['keys_outlier_ratios'] == 1.0


@pytest.mark.parametrize('idx', range(len(ADJ['histograms'])))
def test_adjuster_and_calibration_rules(idx):
    from adacode_b200 import best_bit_analysis_kv_cache as calib
    from adacode_b200 import codec
    e = ADJ['histograms'][idx]
    h = np.asarray(e['hist'], np.int64)
    for impl in (O.choose_params, lambda x: codec.analysis_best_bits(torch.tensor(x))):
        if e['runtime'] is None:
            with pytest.raises(IndexError):
                impl(h)
        else:
            assert list(impl(h)) == e['runtime']
    if e['calibration'] is None:
        with pytest.raises((IndexError, ZeroDivisionError)):
            calib.analysis_best_bits_coo([e['hist']])
    else:
        assert list(O.calibrate_coo(h)) == e['calibration']
        r, n = calib.analysis_best_bits_coo([e['hist']])
        assert [r[0], n[0]] == e['calibration']


def test_calibration_json_consumer(tmp_path):
    from adacode_b200 import export_initial_compress_parameters, model_config_map
    gold = os.path.join(HERE, 'golden')
    rights, nbits = export_initial_compress_parameters(os.path.join(gold, 'calibration_kv.json'))
    assert [list(r) for r in rights] == ADJ['calibration_kv']['rights']
    assert [list(n) for n in nbits] == ADJ['calibration_kv']['nbits']
    rights, nbits = export_initial_compress_parameters(os.path.join(gold, 'calibration_mla.json'))
    assert [list(r) for r in rights] == ADJ['calibration_mla']['rights']
    assert [list(n) for n in nbits] == ADJ['calibration_mla']['nbits']
    cfg = model_config_map['qwen3_4B_config'](kv_cache_path=os.path.join(gold, 'calibration_kv.json'))
    assert cfg.block_size == 128 and cfg.model_id.endswith('Qwen/Qwen3-4B')
    assert [list(r) for r in cfg.rights] == ADJ['calibration_kv']['rights']
    with pytest.raises(FileNotFoundError):
        model_config_map['mistral_7B_config'](kv_cache_path=str(tmp_path / 'missing.json'))
    bad = tmp_path / 'bad.json'
    bad.write_text('{"c4": {"0": {"prefill_q": []}}}')
    with pytest.raises(KeyError):
        export_initial_compress_parameters(str(bad))


def test_library_exports_every_declared_symbol():
    from adacode_b200 import _lib
    from adacode_b200.build import LIB_PATH
    header = open(os.path.join(ROOT, 'include', 'adacode.h')).read()
    declared = set(re.findall(r'\b(adacode_[a-z0-9_]+)\s*\(', header))
    assert declared, 'no declarations found in include/adacode.h'
    lib = ctypes.CDLL(LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f'{name} declared in adacode.h but not exported'
    assert declared == set(_lib.EXPORTED_SYMBOLS)
    assert _lib.lib().adacode_version() >= 100
    assert _lib.lib().adacode_strerror(-3).decode() == 'workspace too small'


def test_no_cpu_fallback():
    from adacode_b200 import codec
    x = torch.zeros((1, 1, 128, 16), dtype=torch.bfloat16)
    with pytest.raises(Exception) as ei:
        codec.compress_tiled_tensor(x, right=129, nbits=3)
    assert 'CUDA' in str(ei.value) or 'cuda' in str(ei.value)
    # nothing under the package imports the oracle
    pkg = os.path.join(ROOT, 'adacode_b200')
    for fn in os.listdir(pkg):
        if fn.endswith('.py'):
            src = open(os.path.join(pkg, fn)).read()
            assert 'import oracle' not in src and 'from oracle' not in src, fn

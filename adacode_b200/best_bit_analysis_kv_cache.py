"""Calibration consumer: exponent-histogram JSON -> initial (right, nbits) per layer.

Drop-in for the part of the reference's ``best_bit_analysis_kv_cache.py`` that the cache path
uses (``export_initial_compress_parameters`` and what it calls).  JSON schema, as written by
the reference's exporter (export_kvcache_status.py:283-296, :423-424)::

    {dataset: {layer_idx_str: {"prefill_keys": [256 ints], "decode_keys": [...],
                                "prefill_values": [...], "decode_values": [...]}}}

MLA files use ``latent`` / ``rope`` in place of ``keys`` / ``values``
(rename_mla_cache_stats.py:7-24).  The ranking itself runs in the C library
(``adacode_calibrate_host``) so that host and device share one implementation of the rule.
"""
from __future__ import annotations

import ctypes
import json

from . import _lib


def _resolve_component_names(freq_dict):
    """reference: best_bit_analysis_kv_cache.py:101-110."""
    if 'prefill_keys' in freq_dict and 'prefill_values' in freq_dict:
        return 'keys', 'values'
    if 'prefill_latent' in freq_dict and 'prefill_rope' in freq_dict:
        return 'latent', 'rope'
    raise KeyError(
        'Cannot resolve cache component names from frequency dict. '
        f'Expected keys/values or latent/rope fields, got {sorted(freq_dict.keys())}')


def get_freq_by_keys(freq_dict, prefix_key):
    """Histograms of the two cached tensors for one stage (reference: :112-123);
    ``'merge'`` adds prefill and decode bin by bin."""
    first, second = _resolve_component_names(freq_dict)
    if prefix_key == 'merge':
        keys = [p + d for p, d in zip(freq_dict[f'prefill_{first}'], freq_dict[f'decode_{first}'])]
        values = [p + d for p, d in zip(freq_dict[f'prefill_{second}'], freq_dict[f'decode_{second}'])]
        return keys, values
    if prefix_key in ('prefill', 'decode'):
        return freq_dict[f'{prefix_key}_{first}'], freq_dict[f'{prefix_key}_{second}']
    raise ValueError(f'unknown infer_stage {prefix_key!r}')


def _calibrate_one(hist) -> tuple:
    if len(hist) != 256:
        raise ValueError(f'expected 256 bins, got {len(hist)}')
    if sum(hist) == 0:
        raise ZeroDivisionError('division by zero')        # the reference divides by the total
    arr = (ctypes.c_int64 * 256)(*[int(v) for v in hist])
    r, n = ctypes.c_int(0), ctypes.c_int(0)
    rc = _lib.lib().adacode_calibrate_host(arr, ctypes.byref(r), ctypes.byref(n))
    if rc == _lib.ERR_NO_CANDIDATE:
        raise IndexError('list index out of range')
    _lib.check(rc, 'adacode_calibrate_host')
    return int(r.value), int(n.value)


def analysis_best_bits_coo(data_lists, titles=None, store_index: bool = False):
    """For each histogram: code lengths 1..8, the 2**n most frequent bins coded, cost
    ``total*n + outliers*8``, first strict minimum wins; ``right`` is the largest coded bin
    (reference: :28-59).  Note that this rule may return n > 4, which the tiled cache rejects."""
    if store_index:
        raise NotImplementedError('store_index=True is not used by the cache path')
    rights, nbits = [], []
    for hist in data_lists:
        r, n = _calibrate_one(hist)
        rights.append(r)
        nbits.append(n)
    return rights, nbits


def export_initial_compress_parameters(json_file_path, dataset_name='c4', infer_stage='merge'):
    """(rights, nbits): one ``(keys, values)`` pair per layer (reference: :191-204)."""
    with open(json_file_path, 'r') as f:
        data = json.load(f)
    layers = list(data[dataset_name].keys())
    per_layer = [get_freq_by_keys(data[dataset_name][str(idx)], infer_stage) for idx in layers]
    keys_rights, keys_nbits = analysis_best_bits_coo([kv[0] for kv in per_layer])
    values_rights, values_nbits = analysis_best_bits_coo([kv[1] for kv in per_layer])
    rights = [(kr, vr) for kr, vr in zip(keys_rights, values_rights)]
    nbits = [(kn, vn) for kn, vn in zip(keys_nbits, values_nbits)]
    return rights, nbits

"""Per-model configuration objects consumed when a cache is built: ``model_id``,
``block_size`` and the calibrated ``rights`` / ``nbits`` read from a calibration JSON.

Drop-in for the KV-cache part of the reference's ``model_configs.py`` (:6-44, :243-253):
``model_config_map[name]()`` returns an object whose ``rights`` and ``nbits`` feed
``Float11Cache(right=..., exp_bits=...)`` (main_lossless_comp.py:112-123).  The reference
writes one near-identical class per model; here one table drives a class factory.  Entries
for weight compression and diffusion models are not part of the cache path and are absent.
"""
from __future__ import annotations

import json
import os

from .best_bit_analysis_kv_cache import export_initial_compress_parameters


class model_default_config:
    """reference: model_configs.py:6-13."""

    def __init__(self):
        self.model_root_dir = '/opt/data/private/'
        self.block_size = 128
        self.config_dict = None
        self.max_new_tokens = 128
        self.compress_text_encoder = False


def convert_json_keys(obj):
    """JSON object keys that look like numbers become numbers, one level deep
    (reference: :15-30)."""
    if isinstance(obj, dict):
        out = {}
        for key, value in obj.items():
            try:
                new_key = float(key) if '.' in key else int(key)
            except (ValueError, AttributeError, TypeError):
                new_key = key
            out[new_key] = value
        return out
    if isinstance(obj, list):
        return [convert_json_keys(item) for item in obj]
    return obj


# registry key -> (hub sub-path under model_root_dir, file stem of its JSONs)
_KV_MODELS = {
    'qwen3_4B_config': ('Qwen/Qwen3-4B', 'Qwen3-4B'),
    'mistral_7B_config': ('mistralai/Mistral-7B-Instruct-v0.3', 'Mistral-7B-Instruct-v0.3'),
    'qwen1p5_moe_config': ('Qwen/Qwen1.5-MoE-A2.7B-Chat', 'Qwen1.5-MoE-A2.7B-Chat'),
    'huihui_moe_config': ('huihui-ai/Huihui-MoE-1.2B-A0.6B', 'Huihui-MoE-1.2B-A0.6B'),
    'qwen2_14B_config': ('Qwen/Qwen2.5-14B-Instruct', 'Qwen2.5-14B-Instruct'),
    'llama_3p1_8B_config': ('LLM-Research/Meta-Llama-3.1-8B-Instruct', 'Meta-Llama-3.1-8B-Instruct'),
    'phi_4_config': ('LLM-Research/Phi-4-reasoning-plus', 'Phi-4-reasoning-plus'),
    'ds_dis_llama_8b_config': ('deepseek-ai/DeepSeek-R1-Distill-Llama-8B', 'DeepSeek-R1-Distill-Llama-8B'),
    'ds_dis_qwen_7b_config': ('deepseek-ai/DeepSeek-R1-Distill-Qwen-7B', 'DeepSeek-R1-Distill-Qwen-7B'),
    'deepseek_v2_lite_config': ('deepseek-ai/DeepSeek-V2-Lite', 'DeepSeek-V2-Lite'),
}


def _make_config_class(name: str, hub_path: str, stem: str):
    default_weights = f'./model_configs/{stem}_weights.json'
    default_kv = f'./model_configs/kv_test_{stem}_exp.json'

    def __init__(self, config_path=default_weights, kv_cache_path=default_kv):
        model_default_config.__init__(self)
        self.model_id = f'{self.model_root_dir}/{hub_path}'
        if os.path.exists(config_path):
            with open(config_path, 'r', encoding='utf-8') as f:
                self.config_dict = convert_json_keys(json.load(f))
        # a missing calibration file raises FileNotFoundError, as in the reference (:44)
        self.rights, self.nbits = export_initial_compress_parameters(kv_cache_path)

    return type(name, (model_default_config,), {'__init__': __init__, '__doc__': f'Cache settings of {stem}.'})


def default_kv_calibration_path(name: str) -> str:
    """Where ``model_config_map[name]()`` looks for the calibration JSON of that model."""
    return f'./model_configs/kv_test_{_KV_MODELS[name][1]}_exp.json'


model_config_map = {name: _make_config_class(name, *spec) for name, spec in _KV_MODELS.items()}
globals().update(model_config_map)

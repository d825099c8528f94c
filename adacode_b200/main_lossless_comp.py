"""Command-line runner of generation with a lossless KV cache, argument for argument the part
of the reference's ``main_lossless_comp.py`` that serves ``--kv_cache_impl dynamic | float11 |
mla_float11`` (:101-149 cache construction, :161-185 synthetic inputs, :216-290 flags,
:342-458 the per-batch record written to ``--output_path``).

    python -m adacode_b200.main_lossless_comp --model_config_name llama_3p1_8B_config \\
        --kv_cache_impl float11 --float11_need_adjust --float11_update_steps 128 \\
        --use_synthetic_data --synthetic_seq_length 4096 --batch_size 32 --num_seqence 32 \\
        --max_new_tokens 128 --min_new_tokens 128 --random_init

Two things the reference takes from files that do not ship with it are made here instead when
``--random_init`` is given: the checkpoint (random bf16 weights of the named architecture,
``--random_init_seed``) and the calibration JSON (exponent histograms of the K/V of a short
synthetic prompt through ``export_kvcache_status.extract_exp_freq``, written to the path the
model config reads).  Without ``--random_init`` the model is loaded with ``from_pretrained`` and
the calibration JSON must exist, as in the reference.

Not provided (other subsystems of the reference): ``cpu_offload`` and ``nvcomp_ans`` caches,
``--compress_weights``, dataset loaders (only ``--use_synthetic_data`` inputs).
``--fused_decode`` (no reference counterpart) serves decode steps with the fused attention kernel.
"""
from __future__ import annotations

import argparse
import json
import os
import time
from pathlib import Path

import torch

# architectures for --random_init: what AutoConfig would read from the checkpoints the registry names
ARCHITECTURES = {
    'llama_3p1_8B_config': ('llama', dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                                          num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                                          vocab_size=128256, rope_theta=500000.0, rms_norm_eps=1e-5)),
    'ds_dis_llama_8b_config': ('llama', dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                                             num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                                             vocab_size=128256, rope_theta=500000.0, rms_norm_eps=1e-5)),
    'qwen3_4B_config': ('qwen3', dict(hidden_size=2560, intermediate_size=9728, num_hidden_layers=36,
                                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936,
                                      rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True)),
    'mistral_7B_config': ('mistral', dict(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                                          num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                                          vocab_size=32768, rope_theta=1000000.0, rms_norm_eps=1e-5)),
    'deepseek_v2_lite_config': ('deepseek_v2', dict(hidden_size=2048, intermediate_size=10944, num_hidden_layers=27,
                                                    num_attention_heads=16, num_key_value_heads=16, kv_lora_rank=512,
                                                    q_lora_rank=None, qk_rope_head_dim=64, qk_nope_head_dim=128,
                                                    v_head_dim=128, vocab_size=102400, n_routed_experts=64,
                                                    n_shared_experts=2, num_experts_per_tok=6,
                                                    moe_intermediate_size=1408, first_k_dense_replace=1)),
}


def _resolve_kv_cache_impl(args) -> str:
    """reference: :86-98."""
    if args.kv_cache_impl != 'auto':
        return args.kv_cache_impl
    if args.compress_kv_cache:
        return 'float11'
    return 'dynamic'


def _build_kv_cache(args, model, model_config, kv_cache_impl: str):
    """reference: :101-149 (the caches of this package only)."""
    from transformers import DynamicCache
    from .float_cache_utils import Float11Cache
    from .mla_float_cache_utils import MLAFloat11Cache
    if kv_cache_impl == 'dynamic':
        return DynamicCache(config=model.config)
    if kv_cache_impl == 'float11':
        return Float11Cache(
            config=model.config, right=model_config.rights, exp_bits=model_config.nbits,
            need_adjust=bool(args.float11_need_adjust), update_steps=int(args.float11_update_steps),
            residual_length=0, block_size=int(args.block_size), layout=args.float11_layout,
            seq_tile_size=args.float11_seq_tile_size)
    if kv_cache_impl == 'mla_float11':
        return MLAFloat11Cache(
            config=model.config, right=model_config.rights, exp_bits=model_config.nbits,
            latent_right=int(args.mla_latent_right), rope_right=int(args.mla_rope_right),
            latent_nbits=int(args.mla_latent_nbits), rope_nbits=int(args.mla_rope_nbits),
            need_adjust=bool(args.float11_need_adjust), update_steps=int(args.float11_update_steps),
            residual_length=0, block_size=int(args.block_size), layout=args.float11_layout,
            seq_tile_size=args.float11_seq_tile_size, mla_cache_mode=args.mla_cache_mode,
            validate_shapes=not bool(args.disable_mla_shape_check),
            compress_rope=not bool(args.mla_disable_rope_compression))
    raise ValueError(f'Unsupported kv_cache_impl: {kv_cache_impl} (this package provides dynamic, float11, mla_float11)')


def _model_primary_device(model) -> torch.device:
    return next(model.parameters()).device


def _make_synthetic_inputs(args, model, batch_size: int, start_idx: int, special_ids=()) -> dict:
    """reference: :161-185."""
    seq_length = max(1, int(args.synthetic_seq_length))
    vocab_size = int(model.config.get_text_config(decoder=True).vocab_size)
    device = _model_primary_device(model)
    if args.synthetic_token_id is not None:
        token_id = int(args.synthetic_token_id)
        if token_id < 0 or token_id >= vocab_size:
            raise ValueError(f'--synthetic_token_id must be in [0, {vocab_size}), got {token_id}.')
        input_ids = torch.full((batch_size, seq_length), token_id, dtype=torch.long, device=device)
    else:
        low = 3 if vocab_size > 4 else 0
        generator = torch.Generator(device='cpu')
        generator.manual_seed(int(args.synthetic_seed) + int(start_idx))
        input_ids = torch.randint(low=low, high=vocab_size, size=(batch_size, seq_length), dtype=torch.long,
                                  generator=generator).to(device)
        for special_id in special_ids:
            if special_id is not None and 0 <= int(special_id) < vocab_size:
                input_ids.masked_fill_(input_ids == int(special_id), low)
    attention_mask = torch.ones((batch_size, seq_length), dtype=torch.long, device=device)
    return {'input_ids': input_ids, 'attention_mask': attention_mask}


def _sanitize_for_json(obj):
    if isinstance(obj, dict):
        return {str(k): _sanitize_for_json(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_sanitize_for_json(v) for v in obj]
    if isinstance(obj, torch.Tensor):
        return obj.tolist()
    if isinstance(obj, (torch.device, torch.dtype)):
        return str(obj)
    return obj


def build_random_model(name: str, device, seed: int = 0, num_hidden_layers=None):
    """Random bf16 weights of the architecture registered under ``name``."""
    import transformers
    if name not in ARCHITECTURES:
        raise ValueError(f'no architecture registered for {name!r}: known {sorted(ARCHITECTURES)}')
    kind, fields = ARCHITECTURES[name]
    fields = dict(fields)
    if num_hidden_layers:
        fields['num_hidden_layers'] = int(num_hidden_layers)
    cfg_cls = {'llama': 'LlamaConfig', 'qwen3': 'Qwen3Config', 'mistral': 'MistralConfig',
               'deepseek_v2': 'DeepseekV2Config'}[kind]
    cfg = getattr(transformers, cfg_cls)(**fields)
    torch.manual_seed(int(seed))
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(device):
            model = transformers.AutoModelForCausalLM.from_config(cfg)
    finally:
        torch.set_default_dtype(prev)
    return model.eval()


def write_calibration_json(model, path: str, seq_len: int = 512, batch: int = 2, seed: int = 1) -> None:
    """Exponent histograms of the K/V a short synthetic prompt leaves in a ``DynamicCache``, in the
    layout ``export_initial_compress_parameters`` reads (dataset key 'c4', decode histograms zero)."""
    from transformers import DynamicCache
    from .export_kvcache_status import extract_exp_freq
    vocab = int(model.config.get_text_config(decoder=True).vocab_size)
    ids = torch.randint(3, vocab, (batch, seq_len), generator=torch.Generator('cpu').manual_seed(seed))
    cache = DynamicCache(config=model.config)
    with torch.no_grad():
        model(ids.to(_model_primary_device(model)), past_key_values=cache, use_cache=True, logits_to_keep=1)
    freq = extract_exp_freq(cache, prefill_len=seq_len)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    Path(path).write_text(json.dumps({'c4': {str(k): v for k, v in freq.items()}}), encoding='utf-8')


def get_parse() -> argparse.ArgumentParser:
    """reference: :216-290 (flags of the subsystems this package does not provide are accepted and refused)."""
    p = argparse.ArgumentParser(description='Run generation with a lossless KV cache.')
    p.add_argument('--model_config_name', type=str, default='qwen2_14B_config')
    p.add_argument('--compress_weights', action='store_true')
    p.add_argument('--compress_kv_cache', action='store_true',
                   help='Compatibility flag: use Float11Cache when kv_cache_impl=auto.')
    p.add_argument('--kv_cache_impl', type=str, default='auto',
                   choices=('auto', 'dynamic', 'cpu_offload', 'float11', 'mla_float11', 'nvcomp_ans'))
    p.add_argument('--block_size', type=int, default=128)
    p.add_argument('--float11_layout', '--kv_layout', type=str, default='segmented_tiled',
                   choices=('legacy', 'tiled', 'segmented_tiled'), dest='float11_layout')
    p.add_argument('--float11_need_adjust', '--kv_adjuster_enabled', action='store_true', dest='float11_need_adjust')
    p.add_argument('--float11_update_steps', '--kv_adjust_update_steps', type=int, default=64,
                   dest='float11_update_steps')
    p.add_argument('--float11_seq_tile_size', type=int, default=None)
    p.add_argument('--mla_cache_mode', type=str, default='auto', choices=('auto', 'latent', 'expanded'))
    p.add_argument('--mla_latent_right', type=int, default=127)
    p.add_argument('--mla_rope_right', type=int, default=127)
    p.add_argument('--mla_latent_nbits', type=int, default=4)
    p.add_argument('--mla_rope_nbits', type=int, default=4)
    p.add_argument('--mla_disable_rope_compression', action='store_true')
    p.add_argument('--disable_mla_shape_check', action='store_true')
    p.add_argument('--max_new_tokens', type=int, default=None)
    p.add_argument('--min_new_tokens', type=int, default=0)
    p.add_argument('--do_sample', action='store_true')
    p.add_argument('--num_seqence', type=int, default=64)
    p.add_argument('--batch_size', type=int, default=1)
    p.add_argument('--max_length', type=int, default=20480)
    p.add_argument('--datasets', '--dataset', nargs='+', default=None)
    p.add_argument('--use_synthetic_data', action='store_true')
    p.add_argument('--synthetic_seq_length', type=int, default=2048)
    p.add_argument('--synthetic_token_id', type=int, default=None)
    p.add_argument('--synthetic_seed', type=int, default=0)
    p.add_argument('--output_path', type=str, default=None)
    # additions of this package
    p.add_argument('--random_init', action='store_true',
                   help='random bf16 weights of the named architecture and a calibration JSON made on the spot')
    p.add_argument('--random_init_seed', type=int, default=0)
    p.add_argument('--random_init_layers', type=int, default=None, help='fewer decoder layers (smoke runs)')
    p.add_argument('--fused_decode', action='store_true',
                   help='float11 only: decode steps through the fused unpack + attention kernel')
    return p


def run(args) -> dict:
    from transformers import GenerationConfig
    from .model_configs import default_kv_calibration_path, model_config_map
    if args.compress_weights:
        raise NotImplementedError('--compress_weights belongs to the weight-compression subsystem, not to the cache path')
    kv_cache_impl = _resolve_kv_cache_impl(args)
    if kv_cache_impl in ('cpu_offload', 'nvcomp_ans'):
        raise NotImplementedError(f'--kv_cache_impl {kv_cache_impl} is a comparator cache of the reference, not provided')
    dataset_names = args.datasets or (['synthetic'] if args.use_synthetic_data else ['longbench'])
    if dataset_names != ['synthetic']:
        raise NotImplementedError('only --use_synthetic_data inputs are provided (the datasets are not redistributable)')

    device = torch.device('cuda', torch.cuda.current_device())
    config_cls = model_config_map[args.model_config_name]
    tokenizer = None
    if args.random_init:
        model = build_random_model(args.model_config_name, device, args.random_init_seed, args.random_init_layers)
        kv_path = default_kv_calibration_path(args.model_config_name)
        stem = os.path.basename(kv_path)[len('kv_test_'):-len('_exp.json')]
        if kv_cache_impl != 'dynamic' and not os.path.exists(kv_path):
            write_calibration_json(model, kv_path)
        model_config = config_cls(kv_cache_path=kv_path) if kv_cache_impl != 'dynamic' else None
        model_id = stem
    else:
        from transformers import AutoModelForCausalLM, AutoTokenizer
        model_config = config_cls()
        model_id = model_config.model_id
        model = AutoModelForCausalLM.from_pretrained(model_id, dtype=torch.bfloat16, device_map='auto').eval()
        tokenizer = AutoTokenizer.from_pretrained(model_id)
        if tokenizer.pad_token is None:
            tokenizer.pad_token = tokenizer.eos_token
    if model_config is not None:
        # the calibration rule may ask for more than 4 bits, which the tiled cache rejects: clamp as the
        # run-time adjuster would (n in 2..4 with an escape slot)
        model_config.nbits = [tuple(min(int(n), 4) for n in pair) for pair in model_config.nbits]
    max_new_tokens = args.max_new_tokens if args.max_new_tokens is not None else (
        model_config.max_new_tokens if model_config is not None else 128)
    output_path = args.output_path or f'kv_lossless_{kv_cache_impl}_{model_id.split("/")[-1]}_weights_False_offload_False.json'
    all_info_lists = {}
    if os.path.exists(output_path):
        all_info_lists = json.loads(Path(output_path).read_text(encoding='utf-8'))
    pad_id = tokenizer.pad_token_id if tokenizer is not None else 0
    eos_id = tokenizer.eos_token_id if tokenizer is not None else None
    specials = (pad_id, eos_id, tokenizer.bos_token_id) if tokenizer is not None else ()
    fused = bool(args.fused_decode) and kv_cache_impl == 'float11'
    if fused:
        from . import hf_attention
        model.config._attn_implementation = hf_attention.register()

    dn = 'synthetic'
    all_info_lists[dn] = []
    mini = max(1, int(args.batch_size))
    total_seqs = int(args.num_seqence)
    for start_idx in range(0, total_seqs, mini):
        end_idx = min(start_idx + mini, total_seqs)
        prompt_cache = None
        with torch.no_grad():
            try:
                info = {
                    'dataset': dn, 'sample_start_idx': int(start_idx), 'batch_size': int(end_idx - start_idx),
                    'cache_mode': kv_cache_impl, 'do_sample': bool(args.do_sample), 'max_new_tokens': int(max_new_tokens),
                    'min_new_tokens': int(args.min_new_tokens), 'block_size': int(args.block_size),
                    'input_mode': 'synthetic', 'synthetic_seq_length': int(args.synthetic_seq_length),
                    'synthetic_token_id': args.synthetic_token_id, 'synthetic_seed': int(args.synthetic_seed),
                }
                if kv_cache_impl in ('float11', 'mla_float11'):
                    info.update(float11_layout=args.float11_layout, float11_need_adjust=bool(args.float11_need_adjust),
                                float11_update_steps=int(args.float11_update_steps))
                if kv_cache_impl == 'float11':
                    info['fused_decode'] = fused
                if kv_cache_impl == 'mla_float11':
                    info.update(mla_cache_mode=args.mla_cache_mode, mla_latent_right=int(args.mla_latent_right),
                                mla_rope_right=int(args.mla_rope_right), mla_latent_nbits=int(args.mla_latent_nbits),
                                mla_rope_nbits=int(args.mla_rope_nbits),
                                mla_compress_rope=not bool(args.mla_disable_rope_compression))
                prompt_cache = _build_kv_cache(args, model, model_config, kv_cache_impl)
                new_inputs = _make_synthetic_inputs(args, model, end_idx - start_idx, start_idx, specials)
                input_lengths = new_inputs['attention_mask'].sum(dim=1).float()
                info['input_shape'] = [int(v) for v in new_inputs['input_ids'].shape]
                info['attention_mask_shape'] = [int(v) for v in new_inputs['attention_mask'].shape]
                info['total_input_tokens'] = input_lengths.sum().item()
                info['input_mean_len'] = input_lengths.mean().item()
                generation_config = GenerationConfig(
                    max_new_tokens=max_new_tokens, min_new_tokens=args.min_new_tokens, do_sample=bool(args.do_sample),
                    return_dict_in_generate=True, output_scores=False, output_attentions=False,
                    output_hidden_states=False, pad_token_id=pad_id, eos_token_id=eos_id)
                if not args.do_sample:
                    generation_config.temperature = None
                    generation_config.top_p = None
                    generation_config.top_k = None
                torch.cuda.reset_peak_memory_stats()
                begin = time.time()
                if fused:
                    from . import hf_attention
                    with hf_attention.fused_decode(prompt_cache):
                        outputs = model.generate(**new_inputs, past_key_values=prompt_cache,
                                                 generation_config=generation_config)
                else:
                    outputs = model.generate(**new_inputs, past_key_values=prompt_cache,
                                             generation_config=generation_config)
                torch.cuda.synchronize()
                generate_time = time.time() - begin
                info['generate_time'] = generate_time
                sequences = outputs.sequences if hasattr(outputs, 'sequences') else outputs
                width = int(new_inputs['input_ids'].shape[1])
                head = sequences[:, width:width + 32]
                info['generated_output_head_32'] = ([tokenizer.decode(r, skip_special_tokens=True) for r in head]
                                                    if tokenizer is not None else head.tolist())
                output_lengths = torch.sum(sequences != pad_id, dim=1).float() if tokenizer is not None else \
                    torch.full((sequences.shape[0],), float(sequences.shape[1]))
                info['total_output_tokens'] = output_lengths.sum().item()
                info['output_mean_len'] = output_lengths.mean().item()
                info['total_new_tokens'] = info['total_output_tokens'] - info['total_input_tokens']
                info['tokens_per_second'] = info['total_new_tokens'] / generate_time if generate_time > 0 else 0.0
                if hasattr(prompt_cache, 'get_memory'):
                    info.update(prompt_cache.get_memory())
                info['cuda_peak_allocated_gib'] = sum(
                    torch.cuda.max_memory_allocated(device=torch.device(f'cuda:{i}')) / (1024 ** 3)
                    for i in range(torch.cuda.device_count()))
                all_info_lists[dn].append(_sanitize_for_json(info))
                Path(output_path).write_text(json.dumps(all_info_lists, indent=2), encoding='utf-8')
            finally:
                if hasattr(prompt_cache, 'synchronize_and_release'):
                    prompt_cache.synchronize_and_release()
                del prompt_cache
                torch.cuda.empty_cache()
    return all_info_lists


if __name__ == '__main__':
    os.environ.setdefault('PYTORCH_ALLOC_CONF', 'expandable_segments:True')
    result = run(get_parse().parse_args())
    for rec in result.get('synthetic', []):
        print(json.dumps({k: rec[k] for k in ('cache_mode', 'input_shape', 'tokens_per_second', 'generate_time',
                                              'kv_compressed_memory', 'kv_original_memory') if k in rec}))

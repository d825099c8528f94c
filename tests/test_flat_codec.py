"""The flat layout (``CompressorBitMap``: 'legacy' cache blocks and packed model weights).

CPU: the oracle's tile pack, applied to tiles of one escape-base block each, reproduces the digests
the reference's ``CompressorBitMap.compress`` wrote into ``tests/golden/flat_codec_vectors.json``.
GPU: the CUDA path equals those digests too, round-trips ragged sizes, and the weight hooks of
``manager.convert_model`` leave a model's outputs bit-identical."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import float11_oracle as O
from tests import scenarios, synth

HERE = os.path.dirname(os.path.abspath(__file__))
FLAT = json.load(open(os.path.join(HERE, 'golden', 'flat_codec_vectors.json')))['cases']


def _case_tensor(case):
    n = case['n_elements']
    return synth.kv_tensor((1, 1, n // 8, 8), seed=case['seed'], key_offset=bool(case['seed'] & 1)).reshape(-1)


def _oracle_flat(x, right, nbits, ibs):
    """Flat pack through the oracle: whole blocks as tiles; a ragged end is padded with zeros whose
    escapes (the last ones of the stream) are dropped again."""
    n = x.numel()
    u = O.as_u16(x.view(1, 1, -1, 8)).reshape(-1)
    pad = (-n) % ibs
    left = right - 2 ** nbits + 1
    up = np.concatenate([u, np.zeros(pad, np.uint16)])
    p = O.pack_block(up.reshape(1, up.size // ibs, ibs // 8, 8), right, nbits, need_hist=True)
    base = p.tile_invalid_base.astype(np.int64)
    esc = p.invalid_exp
    hist = p.hist.copy()
    if pad:
        e = (u[(n // ibs) * ibs:] >> 7) & 0xFF
        real = int(((e <= left) | (e > right)).sum())
        keep = (int(base[-2]) if base.size > 1 else 0) + real
        esc = esc[:keep]
        base[-1] = keep
        hist[0] -= pad
    return p.sign_mass_data[:n], p.exp_data[: n * nbits // 8], esc, base, hist


@pytest.mark.parametrize('case', FLAT, ids=lambda c: f"n{c['n_elements']}_b{c['nbits']}")
def test_oracle_reproduces_reference_flat_pack(case):
    x = _case_tensor(case)
    sm, cd, esc, base, hist = _oracle_flat(x, case['right'], case['nbits'], case['invalid_block_size'])
    assert case['block_base_dtype'] == 'torch.int64'
    assert scenarios._sha(sm) == case['sign_mass_data'] and scenarios._sha(cd) == case['exp_data']
    assert scenarios._sha(esc) == case['invalid_exp'] and esc.size == case['n_escapes']
    assert scenarios._sha(base) == case['block_base']
    assert [int(v) for v in hist] == case['hist']
    assert sm.size + cd.size + esc.size + 8 * base.size == case['compressed_memory']


@pytest.mark.gpu
@pytest.mark.parametrize('case', FLAT, ids=lambda c: f"n{c['n_elements']}_b{c['nbits']}")
def test_cuda_flat_pack_matches_reference_digests(cuda_device, case):
    from adacode_b200 import codec
    from adacode_b200.compress_bitmap_merge import CompressorBitMap
    x = _case_tensor(case)
    c, hist = CompressorBitMap.compress_block(x.to(cuda_device), case['right'], case['nbits'], need_adjust=True)
    assert c.invalid_block_size == case['invalid_block_size'] and str(c.block_base.dtype) == case['block_base_dtype']
    assert scenarios._sha(c.sign_mass_data) == case['sign_mass_data'] and scenarios._sha(c.exp_data) == case['exp_data']
    assert scenarios._sha(c.invalid_exp) == case['invalid_exp'] and scenarios._sha(c.block_base) == case['block_base']
    assert hist.cpu().tolist() == case['hist']
    assert c.get_memory()['compressed_memory'] == case['compressed_memory']
    back = c.uncompress()
    assert torch.equal(back.cpu().view(torch.int16), x.view(torch.int16))
    again = CompressorBitMap.from_state(c.export_state()).materialize()
    assert torch.equal(again, back)
    dense = c.update_compress(case['right'] + 1, case['nbits'])
    assert torch.equal(dense, back) and c.sign_mass_data is None and c.right == case['right'] + 1
    codec.check_device_status(cuda_device)


@pytest.mark.gpu
def test_flat_unpack_of_a_large_tensor_uses_big_tiles(cuda_device):
    """More than 16384 elements: most of the tensor is decoded as 128 x 128 tiles that take every
    16th (8th, 64th) block base; the rest block by block; a ragged end through a padded copy."""
    from adacode_b200.compress_bitmap_merge import CompressorBitMap
    for nbits, n in ((3, 5 * 16384 + 3 * 1024 + 8 * 50), (4, 3 * 16384 + 256 * 7), (2, 2 * 16384), (1, 16384 + 1024)):
        x_cpu = synth.inject_escapes(synth.kv_tensor((1, 1, n // 8, 8), seed=n % 97, s=2.0), seed=3, left=120,
                                     right=128, p_window=0.05).reshape(-1)
        c = CompressorBitMap(right=129, nbits=nbits)
        c.compress(x_cpu.to(cuda_device))
        sm, cd, esc, base, _ = _oracle_flat(x_cpu, 129, nbits, c.invalid_block_size)
        assert np.array_equal(c.sign_mass_data.cpu().numpy(), sm) and np.array_equal(c.exp_data.cpu().numpy(), cd)
        assert np.array_equal(c.invalid_exp.cpu().numpy(), esc) and np.array_equal(c.block_base.cpu().numpy(), base)
        out = torch.empty(n, dtype=torch.int16, device=cuda_device)
        c.uncompress_with_weights(out)
        assert torch.equal(out.cpu(), x_cpu.view(torch.int16))


@pytest.mark.gpu
def test_weight_hooks_keep_model_outputs_bit_identical(cuda_device):
    """``convert_model``: the decoder layers' and the (tied) embedding's parameters live packed; each
    forward decodes them just in time and drops the dense views again."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from adacode_b200 import manager
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=64, vocab_size=1024, max_position_embeddings=128,
                      tie_word_embeddings=True)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).to(cuda_device).eval()
    ids = torch.randint(0, 1024, (2, 40), device=cuda_device)
    with torch.no_grad():
        want = model(ids).logits.clone()
    blocks = {0: ('model.embed_tokens', 'model.embed_tokens', ['model.embed_tokens.weight'])}
    for l in range(cfg.num_hidden_layers):
        prefix = f'model.layers.{l}'
        names = [n for n, _ in model.named_parameters() if n.startswith(prefix + '.')]
        blocks[l + 1] = (prefix, prefix, names)
    config = manager.build_block_config(model, blocks)
    dense_bytes = sum(p.numel() * 2 for p in model.parameters())
    manager.convert_model(model, config, is_tie_weight=True, release_hook=True)
    assert not any(n.startswith('model.layers.') for n, _ in model.named_parameters())
    packed = sum(model.get_submodule(spec['decode_hook_name']).compressor.get_memory()['compressed_memory']
                 for spec in config.values())
    assert packed < 0.85 * dense_bytes
    with torch.no_grad():
        for _ in range(2):                               # every forward decodes again
            got = model(ids).logits
            assert torch.equal(got, want)
    assert 'weight' not in model.model.layers[0].self_attn.q_proj.__dict__       # released after the forward

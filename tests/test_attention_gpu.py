"""Fused unpack + decode attention (``adacode_decode_attn``) against an fp32 PyTorch attention
over the same (losslessly cached) K and V.

This is floating-point work, so the bar is a tolerance, not bit equality.  The kernels accumulate
in fp32 and round the result to bf16 once; for head_dim 128 the probabilities are rounded to bf16
before the tensor-core product (numerator and denominator alike).  Expected error: one bf16
rounding of the output (relative 2**-9), the probabilities' rounding (2**-9 each, mostly
cancelling), fp32 summation order and fast-exp noise:
``|out - ref| <= 2**-8 * |ref| + 2e-3 * max|ref|`` is asserted for every output element.
"""
import math

import pytest
import torch

from tests import synth
from tests.scenarios import StubConfig

pytestmark = pytest.mark.gpu

RTOL = 2.0 ** -8
ATOL_FRAC = 2e-3


def _reference(q, k, v, scale):
    """fp32 attention of q [B, Hq, D] over k, v [B, Hkv, S, D] with grouped heads."""
    B, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    kf = k.float().repeat_interleave(G, dim=1)
    vf = v.float().repeat_interleave(G, dim=1)
    scores = torch.einsum('bhd,bhsd->bhs', q.float(), kf) * scale
    return torch.einsum('bhs,bhsd->bhd', torch.softmax(scores, dim=-1), vf)


def _assert_close(out, ref):
    out = out.float()
    bound = RTOL * ref.abs() + ATOL_FRAC * ref.abs().max()
    err = (out - ref).abs()
    worst = (err - bound).max().item()
    assert worst <= 0, f'max excess error {worst:.3e} (max err {err.max().item():.3e}, max ref {ref.abs().max().item():.3e})'


def _pack_mixed(x, params):
    """Pack x [B, H, S, D] block by block, block j with params[j % len(params)] = (right, nbits)."""
    from adacode_b200 import codec
    segs = []
    for j in range(x.shape[2] // 128):
        right, nbits = params[j % len(params)]
        chunk, _ = codec.pack_blocks(x[:, :, j * 128:(j + 1) * 128], right, nbits, 128)
        segs.append(chunk.segment(0))
    return segs


@pytest.mark.parametrize('B,Hq,Hkv,D,n_seg,tail', [
    (1, 8, 8, 128, 3, 0),        # multi-head attention, packed only
    (2, 32, 8, 128, 5, 77),      # grouped queries, ragged dense tail
    (1, 16, 2, 128, 2, 128),     # eight query heads per KV head, full dense block staged
    (3, 4, 4, 64, 4, 1),         # head_dim 64, one dense token
    (1, 8, 2, 64, 0, 200),       # nothing packed yet
    (2, 8, 1, 128, 9, 300),      # multi-query attention, tail longer than two tiles
    (1, 24, 2, 128, 3, 40),      # twelve query heads per KV head: two CTAs along z (8 + 4)
    (1, 16, 1, 64, 2, 10),       # sixteen per KV head, head_dim 64
])
@pytest.mark.parametrize('n_splits', [0, 1, 7])
def test_matches_fp32_attention(cuda_device, B, Hq, Hkv, D, n_seg, tail, n_splits):
    from adacode_b200 import attention, codec
    S = n_seg * 128 + tail
    k_cpu = synth.kv_tensor((B, Hkv, S, D), seed=11, key_offset=True, s=0.5)
    v_cpu = synth.kv_tensor((B, Hkv, S, D), seed=12, s=0.5)
    k, v = k_cpu.to(cuda_device), v_cpu.to(cuda_device)
    g = torch.Generator('cpu').manual_seed(5)
    q = (torch.randn(B, Hq, D, generator=g) * 0.5).to(torch.bfloat16).to(cuda_device)
    scale = 1.0 / math.sqrt(D)
    kseg = _pack_mixed(k[:, :, :n_seg * 128], [(130, 3), (129, 4), (128, 2)])
    vseg = _pack_mixed(v[:, :, :n_seg * 128], [(127, 3), (126, 1), (128, 4)])
    # dense tails live in a larger buffer, as the cache's residual does (non-trivial strides)
    k_tail = v_tail = None
    if tail:
        kbuf = torch.zeros(B, Hkv, tail + 50, D, dtype=torch.bfloat16, device=cuda_device)
        vbuf = torch.zeros_like(kbuf)
        kbuf[:, :, :tail] = k[:, :, n_seg * 128:]
        vbuf[:, :, :tail] = v[:, :, n_seg * 128:]
        k_tail, v_tail = kbuf[:, :, :tail], vbuf[:, :, :tail]
    out = attention.decode_attention(q, kseg, vseg, k_tail, v_tail, scale=scale, n_splits=n_splits)
    codec.check_device_status(cuda_device)
    assert out.shape == q.shape and out.dtype == torch.bfloat16
    _assert_close(out, _reference(q, k, v, scale))


def test_randomised_attention_shapes(cuda_device):
    """Seeded sweep: batch, KV heads, heads per group (also beyond eight), both head sizes, segment
    counts, residual lengths, split counts, code lengths and windows per segment."""
    import numpy as np
    from adacode_b200 import attention, codec
    rng = np.random.default_rng(77)
    for case in range(24):
        B, Hkv = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        G = int(rng.choice([1, 2, 3, 4, 7, 8, 9, 16]))
        D = int(rng.choice([64, 128, 128]))
        n_seg, tail = int(rng.integers(0, 7)), int(rng.integers(0, 260))
        if n_seg == 0 and tail == 0:
            tail = 5
        S = n_seg * 128 + tail
        k = synth.kv_tensor((B, Hkv, S, D), seed=300 + case, key_offset=True, s=0.5).to(cuda_device)
        v = synth.kv_tensor((B, Hkv, S, D), seed=400 + case, s=0.7).to(cuda_device)
        q = (torch.randn(B, Hkv * G, D, generator=torch.Generator('cpu').manual_seed(case)) * 0.5).to(torch.bfloat16).to(cuda_device)
        params = [(int(rng.integers(124, 133)), int(rng.integers(1, 5))) for _ in range(3)]
        kseg = _pack_mixed(k[:, :, :n_seg * 128], params)
        vseg = _pack_mixed(v[:, :, :n_seg * 128], params[::-1])
        k_tail = k[:, :, n_seg * 128:] if tail else None
        v_tail = v[:, :, n_seg * 128:] if tail else None
        scale = float(rng.choice([1.0 / math.sqrt(D), 0.05, 0.3]))
        out = attention.decode_attention(q, kseg, vseg, k_tail, v_tail, scale=scale, n_splits=int(rng.choice([0, 1, 3, 11])))
        _assert_close(out, _reference(q, k, v, scale))
    codec.check_device_status(cuda_device)


def test_escape_heavy_planes_and_peaked_softmax(cuda_device):
    """Windows that miss most exponents (every second element escapes) and scores large enough
    that a handful of tokens carry all the probability mass."""
    from adacode_b200 import attention, codec
    B, Hq, Hkv, D, n_seg = 2, 8, 2, 128, 6
    k_cpu = synth.inject_escapes(synth.kv_tensor((B, Hkv, n_seg * 128, D), seed=3, key_offset=True), 9, 118, 125, p_window=0.01)
    v_cpu = synth.kv_tensor((B, Hkv, n_seg * 128, D), seed=4)
    k, v = k_cpu.to(cuda_device), v_cpu.to(cuda_device)
    # inject_escapes can create huge magnitudes; keep keys finite and moderate for a meaningful softmax
    k = torch.nan_to_num(k.float(), nan=0.0, posinf=0.0, neginf=0.0).clamp(-64, 64).to(torch.bfloat16)
    g = torch.Generator('cpu').manual_seed(6)
    q = (torch.randn(B, Hq, D, generator=g) * 2.0).to(torch.bfloat16).to(cuda_device)
    kseg = _pack_mixed(k, [(125, 2), (121, 1)])
    vseg = _pack_mixed(v, [(124, 1), (127, 2)])
    assert sum(s.invalid_exp.numel() for s in kseg) > 0.2 * k.numel()
    out = attention.decode_attention(q, kseg, vseg, scale=0.25)
    codec.check_device_status(cuda_device)
    _assert_close(out, _reference(q, k, v, 0.25))


def test_cache_decode_attention_follows_update_schedule(cuda_device):
    """``Float11Cache.decode_attention`` must leave the cache in the state ``update`` leaves it in
    (same packed segments, same adjuster decisions) and agree with attention over the dense K/V
    that a twin cache returns from ``update``, step by step across block boundaries."""
    from adacode_b200 import Float11Cache
    B, Hq, Hkv, D, L = 2, 8, 2, 128, 2
    cfg = StubConfig(L)
    kw = dict(need_adjust=True, update_steps=128, block_size=128, layout='segmented_tiled')
    fused = Float11Cache(cfg, 129, 3, **kw)
    dense = Float11Cache(cfg, 129, 3, dense_workspace='layer', **kw)
    prefill = 300
    steps = 140
    k_all = synth.kv_tensor((B, Hkv, prefill + steps, D), seed=21, key_offset=True, s=0.5).to(cuda_device)
    v_all = synth.kv_tensor((B, Hkv, prefill + steps, D), seed=22, s=0.5).to(cuda_device)
    g = torch.Generator('cpu').manual_seed(23)
    qs = (torch.randn(steps, B, Hq, 1, D, generator=g) * 0.5).to(torch.bfloat16).to(cuda_device)
    for layer in range(L):
        fused.update(k_all[:, :, :prefill], v_all[:, :, :prefill], layer)
        dense.update(k_all[:, :, :prefill], v_all[:, :, :prefill], layer)
    scale = 1.0 / math.sqrt(D)
    for t in range(steps):
        pos = prefill + t
        for layer in range(L):
            kt, vt = k_all[:, :, pos:pos + 1], v_all[:, :, pos:pos + 1]
            out = fused.decode_attention(qs[t], kt, vt, layer)
            kd, vd = dense.update(kt, vt, layer)
            assert kd.shape[2] == pos + 1
            _assert_close(out[:, :, 0], _reference(qs[t][:, :, 0], kd, vd, scale))
    for lf, ld in zip(fused.layers, dense.layers):
        assert lf.segment_params() == ld.segment_params()
        assert lf.get_seq_length() == ld.get_seq_length() == prefill + steps
    mf, md = fused.get_memory(), dense.get_memory()
    for key in ('kv_compressed_memory', 'kv_original_memory', 'compressed_block_flushes', 'keys_update_times'):
        assert mf[key] == md[key]
    assert mf['materialize_calls'] == 0


def test_rejects_unsupported_shapes(cuda_device):
    from adacode_b200 import attention
    k96 = synth.kv_tensor((1, 1, 128, 96), seed=1).to(cuda_device)
    q96 = torch.zeros(1, 1, 96, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(ValueError):
        attention.decode_attention(q96, [], [], k96, k96)          # head_dim outside {64, 128}
    q = torch.zeros(1, 6, 128, dtype=torch.bfloat16, device=cuda_device)
    k = synth.kv_tensor((1, 4, 128, 128), seed=1).to(cuda_device)
    with pytest.raises(ValueError):
        attention.decode_attention(q, [], [], k, k)                # 6 query heads on 4 KV heads
    with pytest.raises(ValueError):
        attention.decode_attention(q[:, :1], [], [])               # empty cache


def test_hf_decode_steps_with_fused_attention(cuda_device):
    """A small random-init Llama (head_dim 128, grouped queries) decodes through the fused kernel
    (``hf_attention``): fed the same tokens, the cache follows the same packing schedule as with the
    materialising path, no dense K/V is rebuilt after the prefill, and every step's logits stay
    within 10 % of the logits' spread of the ``DynamicCache`` run (a few bf16 steps of the logits:
    the network runs in bf16 and two attention kernels round differently).  (Free-running greedy tokens are
    not compared: a random-init model's logits are nearly tied, and the fused kernel sums in a
    different order than SDPA, so one flipped arg-max would fork the sequences.)"""
    from transformers import DynamicCache, LlamaConfig, LlamaForCausalLM
    from adacode_b200 import Float11Cache, hf_attention
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=128, vocab_size=1000, max_position_embeddings=1024)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).to(cuda_device).eval()
    ids = torch.randint(0, 1000, (2, 340), device=cuda_device)
    prefill, steps = 200, 140
    ckw = dict(right=129, exp_bits=4, need_adjust=True, update_steps=128, block_size=128, layout='segmented_tiled')

    def run(cache):
        with torch.no_grad():
            logits = [model(ids[:, :prefill], past_key_values=cache, use_cache=True).logits[:, -1].float()]
            for t in range(prefill, prefill + steps):
                logits.append(model(ids[:, t:t + 1], past_key_values=cache, use_cache=True).logits[:, -1].float())
        return torch.stack(logits)

    ref = run(DynamicCache(config=cfg))
    plain = Float11Cache(cfg, **ckw)
    got_plain = run(plain)
    assert torch.equal(ref, got_plain)                       # lossless cache, same attention kernel
    model.config._attn_implementation = hf_attention.register()
    fused = Float11Cache(cfg, **ckw)
    with hf_attention.fused_decode(fused):
        got_fused = run(fused)
    spread = ref.std().item()
    worst = (got_fused - ref).abs().max().item()
    assert worst <= 0.1 * spread, f'max logit difference {worst:.4f} against a spread of {spread:.4f}'
    assert (got_fused.argmax(-1) == ref.argmax(-1)).float().mean().item() >= 0.9
    # same packing schedule (the cached values themselves differ in the last bits from layer 1 on,
    # because they are computed from the previous layer's attention output)
    mp, mf = plain.get_memory(), fused.get_memory()
    for key in ('compressed_block_flushes', 'stored_residual_seq_len', 'stored_compressed_prefix_seq_len'):
        assert mp[key] == mf[key]
    assert abs(mp['kv_compressed_memory'] - mf['kv_compressed_memory']) <= 0.01 * mp['kv_compressed_memory']
    assert mf['materialize_calls'] == 0 and mp['materialize_calls'] > 0
    assert plain.layers[0].segment_params() == fused.layers[0].segment_params()      # layer 0 sees identical K/V


def test_fused_hook_refuses_what_it_cannot_serve(cuda_device):
    """The fused attention function attends to every cached token: a step whose mask hides cached
    positions, a sliding-window layer, or a model left on another attention implementation must
    raise instead of silently computing something else."""
    from adacode_b200 import Float11Cache, hf_attention
    from tests.scenarios import StubConfig
    cache = Float11Cache(StubConfig(1), right=129, exp_bits=4, need_adjust=False, update_steps=0, block_size=128,
                         layout='segmented_tiled')
    k = synth.kv_tensor((2, 2, 200, 128), seed=61, key_offset=True).to(cuda_device)
    v = synth.kv_tensor((2, 2, 200, 128), seed=62).to(cuda_device)
    cache.update(k[:, :, :199], v[:, :, :199], 0)

    class Layer:
        layer_idx = 0
        sliding_window = None

    q = (torch.randn(2, 4, 1, 128, device=cuda_device) * 0.3).to(torch.bfloat16)
    with hf_attention.fused_decode(cache):
        cache.update(k[:, :, 199:], v[:, :, 199:], 0)
        out, _ = hf_attention.float11_fused_attention(Layer(), q, None, None, None, scaling=128 ** -0.5)
        assert out.shape == (2, 1, 4, 128)
        visible = torch.zeros((2, 1, 1, 200), device=cuda_device)
        out2, _ = hf_attention.float11_fused_attention(Layer(), q, None, None, visible, scaling=128 ** -0.5)
        assert torch.equal(out, out2)                      # an all-visible additive mask is fine
        padded = visible.clone()
        padded[0, :, :, :7] = float('-inf')
        with pytest.raises(NotImplementedError, match='hides'):
            hf_attention.float11_fused_attention(Layer(), q, None, None, padded, scaling=128 ** -0.5)
        windowed = Layer()
        windowed.sliding_window = 64
        with pytest.raises(NotImplementedError, match='sliding window'):
            hf_attention.float11_fused_attention(windowed, q, None, None, None, scaling=128 ** -0.5)

    class Cfg:
        _attn_implementation = 'sdpa'

    with pytest.raises(RuntimeError, match='float11_fused'):
        with hf_attention.fused_decode(cache, Cfg()):
            pass

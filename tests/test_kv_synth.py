"""The benchmark's synthetic generator: any slab equals the same region of the whole tensor, and
the CUDA result equals the CPU result bit for bit (the CPU and GPU arms of the benchmark, and the
shards of a multi-GPU run, rely on both)."""
import pytest
import torch

import kv_synth


def _i16(t):
    return t.cpu().contiguous().view(torch.int16)


def test_slabs_tile_the_tensor():
    sigma, offset = kv_synth.channel_tables(4, 64, seed=5, key_offset=True)
    kw = dict(shift_from=200, shift_heads=(2, 3), escapes=(122, 129, 1e-2, 1e-3))
    whole = kv_synth.kv_tensor(9, (3, 4, 384, 64), sigma, offset, **kw)
    part = kv_synth.kv_slab(9, (2, 4, 100, 64), sigma, offset, b0=1, s0=150, **kw)
    assert torch.equal(_i16(part), _i16(whole[1:3, :, 150:250]))
    chunked = kv_synth.kv_tensor(9, (3, 4, 384, 64), sigma, offset, max_elems=1 << 14, **kw)
    assert torch.equal(_i16(chunked), _i16(whole))
    other = kv_synth.kv_tensor(10, (3, 4, 384, 64), sigma, offset, **kw)
    assert not torch.equal(_i16(other), _i16(whole))


def test_distribution_and_escape_rates():
    sigma, offset = kv_synth.channel_tables(8, 128, seed=1)
    x = kv_synth.kv_tensor(3, (2, 8, 1024, 128), sigma, offset)
    z = (x.float() / sigma.view(1, 8, 1, 128)).flatten()
    assert abs(z.mean().item()) < 5e-3 and abs(z.std().item() - 1.0) < 2e-2
    e = kv_synth.kv_tensor(3, (2, 8, 1024, 128), sigma, offset, escapes=(122, 129, 1e-3, 1e-4))
    exp_e = (_i16(e).to(torch.int32) >> 7) & 0xFF
    exp_x = (_i16(x).to(torch.int32) >> 7) & 0xFF
    changed = (exp_e != exp_x)
    assert 0.8e-3 < changed.float().mean().item() < 1.4e-3
    moved = exp_e[changed]
    assert bool(((moved <= 122) | (moved > 129)).all())
    assert 0.5e-4 < ((exp_e == 0) & (exp_x != 0)).float().mean().item() < 2e-4


@pytest.mark.gpu
def test_cuda_bytes_equal_cpu_bytes(cuda_device):
    sigma, offset = kv_synth.channel_tables(8, 128, seed=2, key_offset=True)
    pos = torch.arange(640, dtype=torch.float32).view(640, 1)
    modulation = 1.0 + torch.sin(pos * torch.exp(-torch.arange(128, dtype=torch.float32) / 20.0).view(1, 128))
    for kw in (dict(), dict(shift_from=300, shift_heads=(4, 5, 6, 7), escapes=(123, 130, 1e-2, 1e-3)),
               dict(modulation=modulation)):
        cpu = kv_synth.kv_tensor(21, (2, 8, 640, 128), sigma, offset, 'cpu', b0=3, **kw)
        gpu = kv_synth.kv_tensor(21, (2, 8, 640, 128), sigma, offset, cuda_device, b0=3, **kw)
        assert torch.equal(_i16(gpu), _i16(cpu)), kw.keys()

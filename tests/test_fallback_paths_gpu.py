"""The kernels behind the environment switches: ``ADACODE_DISABLE_PIPELINE=1`` (direct pack /
unpack kernels for every shape) and ``ADACODE_ATTN_SIMPLE=1`` (plain decode attention for
head_dim 128).  The switches are read once per process, so each case runs in a child process
that checks itself against the CPU oracle (bytes) or fp32 attention (tolerance of
tests/test_attention_gpu.py)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_CODEC = r'''
import numpy as np, torch
from adacode_b200 import codec
from oracle import float11_oracle as O
from tests import synth
dev = torch.device('cuda', 0)
for shape, right, nbits in (((2, 4, 256, 128), 130, 3), ((1, 2, 128, 64), 129, 4), ((2, 2, 128, 128), 127, 1)):
    x_cpu = synth.inject_escapes(synth.kv_tensor(shape, seed=5, key_offset=True), seed=6, left=right - 2 ** nbits + 1, right=right)
    x = x_cpu.to(dev)
    chunk, hist = codec.pack_blocks(x, right, nbits, 128, need_hist=True)
    total = np.zeros(256, np.int64)
    for j in range(shape[2] // 128):
        ref = O.pack_block(x_cpu[:, :, j * 128:(j + 1) * 128].contiguous(), right, nbits, need_hist=True)
        seg = chunk.segment(j)
        assert np.array_equal(seg.sign_mass_data.cpu().numpy(), ref.sign_mass_data)
        assert np.array_equal(seg.exp_data.cpu().numpy(), ref.exp_data)
        assert np.array_equal(seg.invalid_exp.cpu().numpy(), ref.invalid_exp)
        assert np.array_equal(seg.tile_invalid_base.cpu().numpy(), ref.tile_invalid_base)
        total += ref.hist
    assert np.array_equal(hist.cpu().numpy().astype(np.int64), total)
    out = torch.zeros_like(x)
    codec.unpack_chunk(chunk, out)
    assert torch.equal(out.cpu().view(torch.int16), x_cpu.view(torch.int16))
    out2 = torch.zeros_like(x)
    codec.unpack_segments(chunk.segments(), out2)
    assert torch.equal(out2.cpu().view(torch.int16), x_cpu.view(torch.int16))
codec.check_device_status(dev)
print('ok')
'''

_ATTN = r'''
import math, torch
from adacode_b200 import attention, codec
from tests import synth
dev = torch.device('cuda', 0)
B, Hq, Hkv, D, n_seg, tail = 2, 8, 2, 128, 4, 70
S = n_seg * 128 + tail
k = synth.kv_tensor((B, Hkv, S, D), seed=11, key_offset=True, s=0.5).to(dev)
v = synth.kv_tensor((B, Hkv, S, D), seed=12, s=0.5).to(dev)
q = (torch.randn(B, Hq, D, generator=torch.Generator('cpu').manual_seed(5)) * 0.5).to(torch.bfloat16).to(dev)
kc, _ = codec.pack_blocks(k[:, :, :n_seg * 128], 130, 3, 128)
vc, _ = codec.pack_blocks(v[:, :, :n_seg * 128], 127, 3, 128)
out = attention.decode_attention(q, kc.segments(), vc.segments(), k[:, :, n_seg * 128:], v[:, :, n_seg * 128:],
                                 scale=1 / math.sqrt(D)).float()
G = Hq // Hkv
kf, vf = k.float().repeat_interleave(G, 1), v.float().repeat_interleave(G, 1)
sc = torch.einsum('bhd,bhsd->bhs', q.float(), kf) / math.sqrt(D)
ref = torch.einsum('bhs,bhsd->bhd', torch.softmax(sc, -1), vf)
assert ((out - ref).abs() <= 2.0 ** -8 * ref.abs() + 2e-3 * ref.abs().max()).all()
codec.check_device_status(dev)
print('ok')
'''


def _run(code: str, **env):
    e = dict(os.environ, **env)
    e['PYTHONPATH'] = ROOT + os.pathsep + e.get('PYTHONPATH', '')
    r = subprocess.run([sys.executable, '-c', code], cwd=ROOT, env=e, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith('ok'), r.stdout[-2000:] + r.stderr[-2000:]


def test_direct_kernels_forced(cuda_device):
    _run(_CODEC, ADACODE_DISABLE_PIPELINE='1')


def test_pipelined_kernels_in_child_process(cuda_device):
    _run(_CODEC)


def test_plain_attention_forced(cuda_device):
    _run(_ATTN, ADACODE_ATTN_SIMPLE='1')

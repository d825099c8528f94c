"""The pack entry point for hosts that cannot allocate device memory
(``adacode_pack_tiles_static``): a serving process that sized all GPU memory at start-up and
forbids later ``cudaMalloc`` calls, or a C program without a tensor library, still has to give
``adacode_pack_tiles`` a scratch buffer — this variant keeps that scratch inside the library.

Checked here, through the C ABI: two calls in a row (different data, different code lengths)
produce exactly the planes, escape stream, tile bases, segment offsets and histogram of the
ordinary entry point; a span too large for the built-in scratch is refused before anything is
launched.  The file name sorts last so that a failure here cannot hide another test's result."""
import ctypes

import pytest
import torch

from tests import synth

pytestmark = pytest.mark.gpu


def _pack(entry, x, right, nbits, workspace):
    """One raw call of `entry` ('plain' or 'static'); returns every output as CPU tensors."""
    from adacode_b200 import _lib
    L = _lib.lib()
    dev = x.device
    B, H, S, D = x.shape
    T = 128
    n_blocks = S // T
    n = x.numel()
    sign = torch.zeros(n, dtype=torch.uint8, device=dev)
    codes = torch.zeros(n * nbits // 8, dtype=torch.uint8, device=dev)
    esc = torch.zeros(n, dtype=torch.uint8, device=dev)
    base = torch.zeros(B * H * n_blocks, dtype=torch.int32, device=dev)
    meta = torch.zeros(n_blocks + 2, dtype=torch.int64, device=dev)      # offsets, then the status word
    hist = torch.zeros(256, dtype=torch.int32, device=dev)
    sb, sh, ss, _ = x.stride()
    stream = torch.cuda.current_stream(dev).cuda_stream
    head = (x.data_ptr(), sb, sh, ss, B, H, n_blocks, T, D, right, nbits, sign.data_ptr(), codes.data_ptr(),
            esc.data_ptr(), esc.numel(), base.data_ptr(), meta.data_ptr(), hist.data_ptr())
    status_ptr = meta.data_ptr() + 8 * (n_blocks + 1)
    if entry == 'static':
        rc = L.adacode_pack_tiles_static(*head, status_ptr, stream)
    else:
        rc = L.adacode_pack_tiles(*head, workspace.data_ptr(), workspace.numel(), status_ptr, stream)
    assert rc == 0, L.adacode_strerror(rc)
    torch.cuda.synchronize(dev)
    total = int(meta[n_blocks].item())
    assert int(meta[n_blocks + 1].item()) == 0, 'device status word set'
    return {'sign': sign.cpu(), 'codes': codes.cpu(), 'esc': esc[:total].cpu(), 'base': base.cpu(),
            'offsets': meta[: n_blocks + 1].cpu(), 'hist': hist.cpu()}


def test_static_scratch_pack_matches_ordinary_pack_twice(cuda_device):
    from adacode_b200 import _lib
    L = _lib.lib()
    cases = [((2, 4, 512, 128), 0, 130, 3), ((1, 8, 1024, 64), 1, 129, 4)]
    for shape, seed, right, nbits in cases:                       # two calls in a row on the shared scratch
        x = synth.inject_escapes(synth.kv_tensor(shape, seed=seed, key_offset=True), seed=seed + 10,
                                 left=right - 2 ** nbits + 1, right=right).to(cuda_device)
        B, H, S, D = shape
        need = L.adacode_pack_workspace_bytes(B * H * (S // 128), 128 * D)
        assert need <= _lib.STATIC_SCRATCH_BYTES
        workspace = torch.zeros(need, dtype=torch.uint8, device=cuda_device)
        got = _pack('static', x, right, nbits, None)
        want = _pack('plain', x, right, nbits, workspace)
        for key in want:
            assert torch.equal(got[key], want[key]), f'{key} differs for {shape}'
        assert int(got['hist'].sum()) == x.numel() and got['esc'].numel() > 0


def test_static_scratch_rejects_oversized_span(cuda_device):
    from adacode_b200 import _lib
    L = _lib.lib()
    B, H, n_blocks, D = 4, 8, 64, 128                              # 33.5 M elements: far beyond the built-in scratch
    assert L.adacode_pack_workspace_bytes(B * H * n_blocks, 128 * D) > _lib.STATIC_SCRATCH_BYTES
    dummy = torch.zeros(64, dtype=torch.uint8, device=cuda_device)
    p = dummy.data_ptr()
    rc = L.adacode_pack_tiles_static(p, 128 * 64 * D, 128 * 64 * D // H, D, B, H, n_blocks, 128, D, 130, 3,
                                     p, p, p, 0, p, p, None, p, torch.cuda.current_stream(cuda_device).cuda_stream)
    assert rc == _lib.ERR_WORKSPACE
    assert L.adacode_strerror(rc).decode() == 'workspace too small'

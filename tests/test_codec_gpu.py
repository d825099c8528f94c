"""GPU parity of the pack / unpack / histogram / adjuster kernels, called through the C ABI
(ctypes), against the CPU oracle on identical seeded inputs.  Bit-exact comparison throughout
(integer/byte work)."""
import numpy as np
import pytest
import torch

from oracle import float11_oracle as O
from tests import synth

pytestmark = pytest.mark.gpu


def _u16(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _check_chunk_against_oracle(chunk, hist, x_cpu, right, nbits, seq_tile):
    B, H, S, D = x_cpu.shape
    total_hist = np.zeros(256, np.int64)
    for j in range(S // seq_tile):
        blk = x_cpu[:, :, j * seq_tile:(j + 1) * seq_tile, :].contiguous()
        ref = O.pack_block(blk, right, nbits, need_hist=True)
        seg = chunk.segment(j)
        assert np.array_equal(seg.sign_mass_data.cpu().numpy(), ref.sign_mass_data), f'sign/mantissa plane, block {j}'
        assert np.array_equal(seg.exp_data.cpu().numpy(), ref.exp_data), f'code plane, block {j}'
        assert np.array_equal(seg.tile_invalid_base.cpu().numpy(), ref.tile_invalid_base), f'tile base, block {j}'
        assert np.array_equal(seg.invalid_exp.cpu().numpy(), ref.invalid_exp), f'escape stream, block {j}'
        assert seg.left == ref.left and seg.get_memory()['compressed_memory'] == ref.compressed_bytes()
        total_hist += ref.hist
    if hist is not None:
        assert np.array_equal(hist.cpu().numpy().astype(np.int64), total_hist)


@pytest.mark.parametrize('nbits', [1, 2, 3, 4])
@pytest.mark.parametrize('shape', [(1, 8, 128, 128), (3, 2, 256, 64), (2, 1, 128, 512), (1, 2, 128, 72), (2, 3, 384, 16)])
def test_pack_matches_oracle_and_round_trips(cuda_device, nbits, shape):
    from adacode_b200 import codec
    x_cpu = synth.kv_tensor(shape, seed=7 + nbits, key_offset=True)
    x = x_cpu.to(cuda_device)
    right = 129
    chunk, hist = codec.pack_blocks(x, right, nbits, 128, need_hist=True)
    _check_chunk_against_oracle(chunk, hist, x_cpu, right, nbits, 128)
    out = torch.zeros_like(x)
    codec.unpack_chunk(chunk, out)
    assert np.array_equal(_u16(out), _u16(x_cpu))
    out2 = torch.zeros_like(x)
    codec.unpack_segments(chunk.segments(), out2)
    assert np.array_equal(_u16(out2), _u16(x_cpu))
    codec.check_device_status(cuda_device)


@pytest.mark.parametrize('nbits,right', [(3, 3), (2, 255), (4, 14), (1, 127), (3, 260)])
def test_all_bf16_patterns_and_extreme_windows(cuda_device, nbits, right):
    """Every bf16 pattern (zeros, subnormals, Inf, NaN) with windows that reach below 0 and
    above 255, where nearly everything escapes (the reference's own fixture uses right=3)."""
    from adacode_b200 import codec
    x_cpu = synth.all_bf16_patterns()
    x = x_cpu.to(cuda_device)
    chunk, hist = codec.pack_blocks(x, right, nbits, 128, need_hist=True)
    _check_chunk_against_oracle(chunk, hist, x_cpu, right, nbits, 128)
    out = torch.zeros_like(x)
    codec.unpack_chunk(chunk, out)
    assert np.array_equal(_u16(out), _u16(x_cpu))
    codec.check_device_status(cuda_device)


def test_strided_source_and_destination(cuda_device):
    """K/V arrive as [B, S, H, D] projections viewed as [B, H, S, D]; the kernels take the strides."""
    from adacode_b200 import codec
    base_cpu = synth.kv_tensor((2, 256, 4, 128), seed=3)          # [B, S, H, D]
    x_cpu = base_cpu.transpose(1, 2)                              # [B, H, S, D] view
    x = base_cpu.to(cuda_device).transpose(1, 2)
    assert not x.is_contiguous()
    chunk, hist = codec.pack_blocks(x, 128, 3, 128, need_hist=True)
    _check_chunk_against_oracle(chunk, hist, x_cpu.contiguous(), 128, 3, 128)
    wide = torch.zeros((2, 4, 256 + 40, 128), dtype=torch.bfloat16, device=cuda_device)
    codec.unpack_chunk(chunk, wide, seq_offset=40)
    assert np.array_equal(_u16(wide[:, :, 40:]), _u16(x_cpu.contiguous()))
    assert int(wide[:, :, :40].abs().sum()) == 0


def test_mixed_segments_one_launch(cuda_device):
    from adacode_b200 import codec
    x_cpu = synth.kv_tensor((2, 4, 384, 128), seed=11)
    x = x_cpu.to(cuda_device)
    params = [(129, 3), (131, 4), (127, 2)]
    segs = []
    for j, (r, n) in enumerate(params):
        seg, _ = codec.compress_tiled_tensor(x[:, :, j * 128:(j + 1) * 128], right=r, nbits=n, seq_tile_size=128)
        ref = O.pack_block(x_cpu[:, :, j * 128:(j + 1) * 128].contiguous(), r, n)
        assert np.array_equal(seg.invalid_exp.cpu().numpy(), ref.invalid_exp)
        assert np.array_equal(seg.exp_data.cpu().numpy(), ref.exp_data)
        segs.append(seg)
    out = torch.zeros_like(x)
    codec.unpack_segments(segs, out)
    assert np.array_equal(_u16(out), _u16(x_cpu))
    # materialize() of a single segment and of its exported state
    one = segs[1].materialize()
    assert np.array_equal(_u16(one), _u16(x_cpu[:, :, 128:256].contiguous()))
    again = codec.materialize_tiled_state(segs[1].export_state())
    assert torch.equal(one, again)


def test_injected_escapes_linear_checksum(cuda_device):
    """Config-4-style escapes (0.1 % out of window, 0.01 % zero/subnormal): byte parity on a
    reduced replica and the size-independent property sum(compressed bytes) == formula."""
    from adacode_b200 import codec
    x_cpu = synth.inject_escapes(synth.kv_tensor((4, 8, 512, 128), seed=5), seed=6, left=122, right=129)
    x = x_cpu.to(cuda_device)
    chunk, hist = codec.pack_blocks(x, 129, 3, 128, need_hist=True)
    _check_chunk_against_oracle(chunk, hist, x_cpu, 129, 3, 128)
    n = x.numel()
    total = sum(chunk.segment(j).get_memory()['compressed_memory'] for j in range(chunk.n_blocks))
    assert total == n + n * 3 // 8 + chunk.n_escapes + 4 * 4 * 8 * chunk.n_blocks
    assert int(hist.sum()) == n


def test_escape_capacity_retry(cuda_device):
    from adacode_b200 import codec
    x_cpu = synth.all_bf16_patterns()
    x = x_cpu.to(cuda_device)
    chunk, _ = codec.pack_blocks(x, 3, 3, 128, escape_capacity=64)     # nearly everything escapes
    ref = O.pack_block(x_cpu, 3, 3)
    assert np.array_equal(chunk.segment(0).invalid_exp.cpu().numpy(), ref.invalid_exp)
    codec.check_device_status(cuda_device)


def test_histogram_kernel(cuda_device):
    from adacode_b200 import codec
    x_cpu = synth.kv_tensor((2, 3, 77, 64), seed=9, key_offset=True)
    h = codec.exponent_hist(x_cpu.to(cuda_device))
    assert np.array_equal(h.cpu().numpy().astype(np.int64), O.exponent_hist(x_cpu))
    strided = x_cpu.to(cuda_device)[:, :, 5:50]
    h2 = codec.exponent_hist(strided)
    assert np.array_equal(h2.cpu().numpy().astype(np.int64), O.exponent_hist(x_cpu[:, :, 5:50].contiguous()))


def test_adjuster_device_and_host(cuda_device):
    from adacode_b200 import codec
    rng = np.random.default_rng(0)
    hists = []
    for i in range(40):
        h = np.zeros(256, np.int64)
        centre = int(rng.integers(100, 140))
        width = int(rng.integers(1, 12))
        idx = np.clip(np.round(rng.normal(centre, width, 20000)).astype(int), 0, 255)
        np.add.at(h, idx, 1)
        if i % 5 == 0:                               # ties and zero-count bins
            h[centre - 1] = h[centre] = h[centre + 1]
        hists.append(h)
    hists.append(np.zeros(256, np.int64))            # nothing seen: no candidate
    hists.append(np.full(256, 10, np.int64))         # flat: no candidate
    dev_out = codec.choose_params_device(torch.tensor(np.stack(hists), dtype=torch.int32, device=cuda_device)).cpu().numpy()
    for h, (r, n) in zip(hists, dev_out):
        try:
            exp = O.choose_params(h)
        except IndexError:
            assert n == 0
            with pytest.raises(IndexError):
                codec.analysis_best_bits(h)
            continue
        assert (int(r), int(n)) == exp
        assert codec.analysis_best_bits(torch.tensor(h)) == exp


def test_argument_errors(cuda_device):
    from adacode_b200 import codec
    x = torch.zeros((1, 2, 128, 64), dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(ValueError):
        codec.compress_tiled_tensor(x, right=129, nbits=5)
    with pytest.raises(ValueError):
        codec.compress_tiled_tensor(x[0], right=129, nbits=3)
    with pytest.raises(ValueError):
        codec.compress_tiled_tensor(x[..., :60], right=129, nbits=3)
    with pytest.raises(ValueError):
        codec.compress_tiled_tensor(x, right=129, nbits=3, seq_tile_size=64)
    with pytest.raises(Exception):
        codec.pack_blocks(x.cpu(), 129, 3)


def test_read_back_matches_cpu_copy(cuda_device):
    """The kernel-written host mailbox returns exactly what a plain device-to-host copy returns."""
    from adacode_b200 import codec
    g = torch.Generator('cpu').manual_seed(3)
    for dtype, shape in ((torch.int64, (163,)), (torch.int32, (2, 256)), (torch.int32, (1,)), (torch.uint8, (64,))):
        t = torch.randint(0, 100, shape, generator=g).to(dtype).to(cuda_device)
        got = codec.read_back(t)
        assert got.shape == tuple(shape) and np.array_equal(got, t.cpu().numpy())
    odd = torch.arange(7, dtype=torch.uint8, device=cuda_device)        # not a multiple of 4 bytes: plain copy
    assert np.array_equal(codec.read_back(odd), odd.cpu().numpy())


def test_pack_pair_equals_two_packs(cuda_device):
    """Keys and values packed with one shared read give the same chunks and histograms as two
    separate ``pack_blocks`` calls, also when the suggested escape capacity is far too small."""
    from adacode_b200 import codec
    k = synth.kv_tensor((2, 4, 384, 128), seed=31, key_offset=True).to(cuda_device)
    v = synth.kv_tensor((2, 4, 384, 128), seed=32).to(cuda_device)
    for caps in ((None, None), (16, 16)):
        kc, vc, kh, vh, kh_host, vh_host = codec.pack_pair(k, v, (129, 3), (127, 2), 128, need_hist=True, capacities=caps)
        for x, chunk, hist, hist_host, (right, nbits) in ((k, kc, kh, kh_host, (129, 3)), (v, vc, vh, vh_host, (127, 2))):
            ref, ref_hist = codec.pack_blocks(x, right, nbits, 128, need_hist=True)
            assert chunk.seg_offsets == ref.seg_offsets
            for a, b in ((chunk.sign_mant, ref.sign_mant), (chunk.codes, ref.codes), (chunk.escapes, ref.escapes),
                         (chunk.tile_base, ref.tile_base), (hist, ref_hist)):
                assert torch.equal(a, b)
            assert np.array_equal(hist_host, ref_hist.cpu().numpy())
    codec.check_device_status(cuda_device)


def test_copy_to_host_refuses_memory_the_device_cannot_address(cuda_device):
    """``adacode_copy_to_host`` only launches towards page-locked host memory: pageable host memory
    and device memory are refused with ADACODE_ERR_INVALID_ARG before any kernel runs."""
    import ctypes
    from adacode_b200 import _lib
    L = _lib.lib()
    src = torch.arange(16, dtype=torch.int32, device=cuda_device)
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    pageable = (ctypes.c_uint32 * 16)()
    assert L.adacode_copy_to_host(src.data_ptr(), ctypes.addressof(pageable), 64, stream) == _lib.ERR_INVALID_ARG
    other = torch.empty(16, dtype=torch.int32, device=cuda_device)
    assert L.adacode_copy_to_host(src.data_ptr(), other.data_ptr(), 64, stream) == _lib.ERR_INVALID_ARG
    pinned = torch.zeros(16, dtype=torch.int32).pin_memory()
    assert L.adacode_copy_to_host(src.data_ptr(), pinned.data_ptr(), 62, stream) == _lib.ERR_INVALID_ARG   # not a multiple of 4
    assert L.adacode_copy_to_host(src.data_ptr(), pinned.data_ptr(), 64, stream) == _lib.OK
    torch.cuda.synchronize(cuda_device)
    assert torch.equal(pinned, src.cpu())


def test_randomised_shapes_windows_and_escape_rates(cuda_device):
    """Seeded sweep over shapes, code lengths, windows and escape rates (from none to nearly all):
    every plane equals the oracle's, both unpack entry points round-trip, also through views of a
    chunk whose escape lists start at arbitrary byte offsets, and pack_pair with tiny capacities."""
    from adacode_b200 import codec
    rng = np.random.default_rng(1234)
    for case in range(60):
        B, H = int(rng.integers(1, 4)), int(rng.integers(1, 5))
        n_blocks = int(rng.integers(1, 5))
        D = int(rng.choice([16, 32, 64, 128, 256]))
        nbits = int(rng.integers(1, 5))
        right = int(rng.integers(118, 136))
        s = float(rng.choice([0.1, 0.5, 1.0, 2.0]))
        x_cpu = synth.kv_tensor((B, H, 128 * n_blocks, D), seed=1000 + case, s=s, key_offset=bool(case & 1))
        if case % 3 == 0:
            x_cpu = synth.inject_escapes(x_cpu, seed=case, left=right - 2 ** nbits + 1, right=right,
                                         p_window=float(rng.choice([1e-3, 0.05, 0.3])), p_zero=1e-3)
        x = x_cpu.to(cuda_device)
        chunk, hist = codec.pack_blocks(x, right, nbits, 128, need_hist=True)
        _check_chunk_against_oracle(chunk, hist, x_cpu, right, nbits, 128)
        out = torch.zeros_like(x)
        codec.unpack_chunk(chunk, out)
        assert np.array_equal(_u16(out), _u16(x_cpu)), f'case {case}: uniform unpack'
        # segments in reverse order into a strided destination: tables with per-segment offsets
        wide = torch.zeros((B, H, 128 * n_blocks + 64, D), dtype=torch.bfloat16, device=cuda_device)
        segs = chunk.segments()[::-1]
        offs = [128 * (n_blocks - 1 - j) for j in range(n_blocks)]
        codec.unpack_segments(segs, wide[:, :, :128 * n_blocks], seq_offsets=offs)
        assert np.array_equal(_u16(wide[:, :, :128 * n_blocks]), _u16(x_cpu)), f'case {case}: segment unpack'
        if case % 5 == 0:
            kc, vc, _, _, _, _ = codec.pack_pair(x, x, (right, nbits), (right - 1, nbits), 128, capacities=(16, 16))
            assert torch.equal(kc.escapes, chunk.escapes) and torch.equal(kc.codes, chunk.codes)
            back = torch.zeros_like(x)
            codec.unpack_chunk(vc, back)
            assert np.array_equal(_u16(back), _u16(x_cpu)), f'case {case}: pair unpack'
    codec.check_device_status(cuda_device)

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
@pytest.mark.parametrize('shape', [(1, 8, 128, 128), (3, 2, 256, 64), (2, 1, 128, 512), (1, 2, 128, 72), (2, 3, 384, 16),
                                   (1, 2, 128, 1024), (1, 1, 128, 1040), (1, 1, 128, 2048)])
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


@pytest.mark.parametrize('D', [128, 64])
def test_pack_jobs_three_tensors_one_launch(cuda_device, D):
    """``adacode_pack_jobs`` through the raw C ABI: three tensors of one shape family (different
    block counts, windows, one without a histogram) in one launch equal three ordinary packs
    (head_dim 64: tiles of 8192 elements, which the pack kernel runs on its 8-warp geometry)."""
    import ctypes
    from adacode_b200 import _lib, codec
    L = _lib.lib()
    B, H, nbits = 2, 3, 3
    specs = [(384, 129, True), (128, 127, False), (256, 131, True)]
    xs = [synth.inject_escapes(synth.kv_tensor((B, H, S, D), seed=70 + i, key_offset=bool(i & 1)), seed=80 + i,
                               left=r - 7, right=r).to(cuda_device) for i, (S, r, _) in enumerate(specs)]
    jobs = (_lib.PackJob * len(specs))()
    outs = []
    n_tiles = 0
    for jb, x, (S, right, want_hist) in zip(jobs, xs, specs):
        nb = S // 128
        n = x.numel()
        o = {'sm': torch.zeros(n, dtype=torch.uint8, device=cuda_device),
             'codes': torch.zeros(n * nbits // 8, dtype=torch.uint8, device=cuda_device),
             'esc': torch.zeros(n, dtype=torch.uint8, device=cuda_device),
             'base': torch.zeros(B * H * nb, dtype=torch.int32, device=cuda_device),
             'off': torch.zeros(nb + 1, dtype=torch.int64, device=cuda_device),
             'hist': torch.zeros(256, dtype=torch.int32, device=cuda_device) if want_hist else None}
        outs.append(o)
        sb, sh, ss, _ = x.stride()
        jb.src_bf16, jb.stride_b, jb.stride_h, jb.stride_s = x.data_ptr(), sb, sh, ss
        jb.n_blocks, jb.right = nb, right
        jb.sign_mant, jb.codes, jb.escapes = o['sm'].data_ptr(), o['codes'].data_ptr(), o['esc'].data_ptr()
        jb.escapes_capacity = n
        jb.tile_base, jb.seg_escape_offsets = o['base'].data_ptr(), o['off'].data_ptr()
        jb.hist256 = o['hist'].data_ptr() if want_hist else 0
        n_tiles += B * H * nb
    ws = torch.zeros(L.adacode_pack_workspace_bytes(n_tiles, 128 * D), dtype=torch.uint8, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    for _ in range(2):                                   # the scratch is left ready for the next call
        for o in outs:
            if o['hist'] is not None:
                o['hist'].zero_()
        rc = L.adacode_pack_jobs(ctypes.addressof(jobs), len(specs), B, H, 128, D, nbits, ws.data_ptr(), ws.numel(),
                                 status.data_ptr(), torch.cuda.current_stream(cuda_device).cuda_stream)
        assert rc == 0, L.adacode_strerror(rc)
        torch.cuda.synchronize(cuda_device)
        assert int(status.item()) == 0
        for o, x, (S, right, want_hist) in zip(outs, xs, specs):
            ref, ref_hist = codec.pack_blocks(x, right, nbits, 128, need_hist=True)
            assert o['off'].cpu().tolist() == ref.seg_offsets
            total = ref.seg_offsets[-1]
            assert torch.equal(o['sm'], ref.sign_mant.reshape(-1)) and torch.equal(o['codes'], ref.codes.reshape(-1))
            assert torch.equal(o['esc'][:total], ref.escapes) and torch.equal(o['base'], ref.tile_base.reshape(-1))
            if want_hist:
                assert torch.equal(o['hist'], ref_hist)
            _check_chunk_against_oracle(ref, ref_hist, x.cpu(), right, nbits, 128)
    assert L.adacode_pack_jobs(ctypes.addressof(jobs), L.adacode_max_jobs() + 1, B, H, 128, D, nbits, ws.data_ptr(),
                               ws.numel(), status.data_ptr(), 0) == _lib.ERR_INVALID_ARG


@pytest.mark.parametrize('D', [128, 96, 512, 64, 1040])
def test_unpack_jobs_and_token_major_destination(cuda_device, D):
    """Keys and values unpacked by one launch (``adacode_unpack_jobs``), the keys into a
    destination whose token rows are not adjacent ([B, S, H, D] memory viewed as [B, H, S, D])."""
    from adacode_b200 import codec
    B, H, S = 2, 3, 384
    k_cpu = synth.kv_tensor((B, H, S, D), seed=41, key_offset=True)
    v_cpu = synth.inject_escapes(synth.kv_tensor((B, H, S, D), seed=42), seed=43, left=121, right=128, p_window=0.2)
    kc, _ = codec.pack_blocks(k_cpu.to(cuda_device), 129, 3, 128)
    vc, _ = codec.pack_blocks(v_cpu.to(cuda_device), 128, 3, 128)
    k_dst = torch.zeros((B, S, H, D), dtype=torch.bfloat16, device=cuda_device).transpose(1, 2)
    v_dst = torch.zeros((B, H, S + 128, D), dtype=torch.bfloat16, device=cuda_device)
    codec.unpack_segments_multi([(kc.segments(), k_dst, None), (vc.segments(), v_dst, None)])
    assert np.array_equal(_u16(k_dst), _u16(k_cpu))
    assert np.array_equal(_u16(v_dst[:, :, :S]), _u16(v_cpu))
    assert int(v_dst[:, :, S:].abs().sum()) == 0
    one = torch.zeros((B, S, H, D), dtype=torch.bfloat16, device=cuda_device).transpose(1, 2)
    codec.unpack_chunk(vc, one)
    assert np.array_equal(_u16(one), _u16(v_cpu))
    codec.check_device_status(cuda_device)


def test_status_word_misaligned_record(cuda_device):
    """A segment record whose plane pointer is off by one byte (inside a valid buffer) is never
    handed to a bulk copy: the call returns, the tile is skipped, the status word says so."""
    from adacode_b200 import _lib, codec
    x_cpu = synth.kv_tensor((1, 2, 256, 128), seed=51)
    chunk, _ = codec.pack_blocks(x_cpu.to(cuda_device), 129, 3, 128)
    segs = chunk.segments()
    table = codec.build_segment_table(segs, None, cuda_device)
    rec = table.view(torch.int64)
    rec[7] += 1                                   # sign_mant pointer of segment 1 (7 int64 words per record)
    out = torch.zeros_like(x_cpu, device=cuda_device)
    codec.unpack_segments(segs, out, table=table)
    with pytest.raises(_lib.AdacodeError, match='not 16-byte aligned'):
        codec.check_device_status(cuda_device)
    assert np.array_equal(_u16(out[:, :, :128]), _u16(x_cpu[:, :, :128].contiguous()))   # segment 0 is untouched by it
    assert int(out[:, :, 128:].abs().sum()) == 0                                          # segment 1 was skipped
    codec.check_device_status(cuda_device)        # the word was cleared; the context is usable
    codec.unpack_segments(segs, out)
    assert np.array_equal(_u16(out), _u16(x_cpu))


def test_status_word_timeout_of_a_bounded_wait(cuda_device):
    """The bounded on-chip wait: with the poll limit lowered and one unit never signalled as
    loaded (``adacode_debug_set_wait_limit``) the launch still ends, reports TIMEOUT and leaves the
    context usable.  Nothing faults or hangs: the withheld unit has nothing to do."""
    from adacode_b200 import _lib, codec
    L = _lib.lib()
    x_cpu = synth.kv_tensor((1, 2, 128, 128), seed=52)
    chunk, _ = codec.pack_blocks(x_cpu.to(cuda_device), 129, 3, 128)
    out = torch.zeros_like(x_cpu, device=cuda_device)
    try:
        L.adacode_debug_set_wait_limit(20000, 0)
        codec.unpack_chunk(chunk, out)
        torch.cuda.synchronize(cuda_device)
    finally:
        L.adacode_debug_set_wait_limit(0, -1)
    with pytest.raises(_lib.AdacodeError, match='bounded on-chip wait'):
        codec.check_device_status(cuda_device)
    out.zero_()
    codec.unpack_chunk(chunk, out)
    assert np.array_equal(_u16(out), _u16(x_cpu))
    codec.check_device_status(cuda_device)


def test_code_counters_are_flushed_on_a_launch_of_very_many_small_tiles(cuda_device):
    """The pack kernel counts codes in 16-bit register fields and empties them every 1024 units.
    A CTA only gets that far with tiny tiles: 640 000 tiles of 128 x 16 elements in one launch give
    each of the 592 CTAs more than 1024 units.  The histogram must equal a plain count."""
    from adacode_b200 import codec
    B, H, blocks, D = 8, 8, 10000, 16
    gen = torch.Generator(device=cuda_device)
    gen.manual_seed(5)
    x = torch.empty((B, H, blocks * 128, D), dtype=torch.bfloat16, device=cuda_device)
    for b in range(B):
        x[b] = (torch.randn((H, blocks * 128, D), generator=gen, device=cuda_device) * 0.7).to(torch.bfloat16)
    want = torch.zeros(256, dtype=torch.int64, device=cuda_device)
    for b in range(B):
        e = (x[b].view(torch.int16).to(torch.int32) >> 7) & 0xFF
        want += torch.bincount(e.flatten(), minlength=256)
    chunk, hist = codec.pack_blocks(x, 127, 3, 128, need_hist=True)
    assert torch.equal(hist.to(torch.int64), want)
    assert chunk.n_escapes == int(want.sum() - want[121:128].sum())
    out = torch.empty_like(x)
    codec.unpack_chunk(chunk, out)
    assert torch.equal(out.view(torch.int16), x.view(torch.int16))
    codec.check_device_status(cuda_device)

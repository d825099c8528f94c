"""Kernel-level timing of pack and unpack on one GPU, for profiling and tuning.

``python microbench.py --shape 16,8,8192,128 --nbits 4 --right 131 --iters 5``

Packs a seeded synthetic K tensor [B, H, S, D] (all S/128 blocks in one launch) and unpacks it
again, timing each kernel with CUDA events on the launching stream (several launches back to
back per sample, so that host launch latency is not counted), and prints one line per
kernel with the algorithmic HBM bytes (2 read + 1 + nbits/8 + p written per element for pack,
the mirror image for unpack, p = escape fraction) divided by the time.  ``--pair`` times a K and a
V tensor of that shape going through ONE launch (``adacode_pack_jobs`` / ``adacode_unpack_jobs``).
Inputs are larger than L2 when the shape is; nothing is copied from or to the host inside the
timed region.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from adacode_b200 import _lib, codec  # noqa: E402


def synthetic_keys(shape, seed: int = 0, device='cuda') -> torch.Tensor:
    """N(0, sigma_c) with sigma_c ~ LogNormal(0, 1), 2 % outlier channels x30 and a per-channel
    offset ~ N(0, 2); a 2048-token slab is generated once and repeated along batch and sequence."""
    B, H, S, D = shape
    g = torch.Generator('cpu').manual_seed(seed)
    base_s = min(S, 2048)
    sigma = torch.exp(torch.randn(H, D, generator=g))
    sigma = torch.where(torch.rand(H, D, generator=g) < 0.02, sigma * 30.0, sigma)
    x = torch.randn(1, H, base_s, D, generator=g) * sigma[None, :, None, :]
    x = (x + (2.0 * torch.randn(H, D, generator=g))[None, :, None, :]).to(torch.bfloat16).to(device)
    reps = (S + base_s - 1) // base_s
    return x.repeat(B, 1, reps, 1)[:, :, :S].contiguous()


def _time(fn, iters: int, warmup: int, inner: int = 8) -> float:
    """Median over ``iters`` samples of the device time of one call of ``fn``.  Each sample times
    ``inner`` calls issued back to back between two events: the host needs tens of microseconds
    to get through the Python and ctypes layers, which a single call between two events would
    count as kernel time (the GPU idles until the launch arrives)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn()                      # keeps the queue non-empty while the first timed call is prepared
        a.record()
        for _ in range(inner):
            fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) / inner)
    times.sort()
    return times[len(times) // 2] * 1e-3


def attention_main(args) -> None:
    """One decode step over a cache of shape --shape for K and for V: the fused kernel reads
    (1 + nbits/8 + p) bytes per cached element; the materialising path reads them too, writes
    2 bytes and lets the attention kernel read 2 bytes again."""
    import torch.nn.functional as F

    from adacode_b200 import attention
    shape = tuple(int(v) for v in args.shape.split(','))
    B, H, S, D = shape
    Hq = args.attention
    dev = torch.device('cuda', 0)
    k = synthetic_keys(shape, seed=0, device=dev)
    v = synthetic_keys(shape, seed=1, device=dev)
    kc, _ = codec.pack_blocks(k, args.right, args.nbits, 128)
    vc, _ = codec.pack_blocks(v, args.right, args.nbits, 128)
    ks, vs = kc.segments(), vc.segments()
    kt = codec.build_segment_table(ks, None, dev)
    vt = codec.build_segment_table(vs, None, dev)
    q = (torch.randn(B, Hq, D, device=dev) * 0.3).to(torch.bfloat16)
    out = torch.empty_like(q)
    dk, dv = torch.empty_like(k), torch.empty_like(v)
    p = (kc.n_escapes + vc.n_escapes) / (2 * k.numel())

    def fused():
        attention.decode_attention(q, ks, vs, key_table=kt, value_table=vt, out=out)

    def materialise():
        codec.unpack_segments(ks, dk, table=kt)
        codec.unpack_segments(vs, dv, table=vt)
        return F.scaled_dot_product_attention(q.unsqueeze(2), dk, dv, enable_gqa=Hq != H)

    def dense_only():
        return F.scaled_dot_product_attention(q.unsqueeze(2), dk, dv, enable_gqa=Hq != H)

    t_f = _time(fused, args.iters, args.warmup)
    t_m = _time(materialise, args.iters, args.warmup)
    t_d = _time(dense_only, args.iters, args.warmup)
    ref = materialise()[:, :, 0].float()
    err = (out.float() - ref).abs().max().item()
    packed_bytes = 2 * k.numel() * (1.0 + args.nbits / 8.0 + p)
    for name, t in (('decode_attn_fused', t_f), ('unpack_then_sdpa', t_m), ('sdpa_on_dense_only', t_d)):
        print(json.dumps({
            'kernel': name, 'shape': list(shape), 'q_heads': Hq, 'nbits': args.nbits, 'escape_fraction': round(p, 5),
            'us': round(t * 1e6, 1), 'packed_GBps': round(packed_bytes / t / 1e9, 1),
            'bf16_equiv_GBps': round(4 * k.numel() / t / 1e9, 1), 'max_abs_diff_vs_sdpa': round(err, 5),
        }))


def pair_main(args) -> None:
    """K and V of one shape through one pack launch and one unpack launch."""
    shape = tuple(int(v) for v in args.shape.split(','))
    B, H, S, D = shape
    dev = torch.device('cuda', 0)
    T = args.seq_tile
    n_blocks = S // T
    xs = [synthetic_keys(shape, seed=i, device=dev) for i in range(2)]
    n = xs[0].numel()
    L = _lib.lib()
    sc = codec._scratch_for(dev)
    ws = sc.workspace_for(2 * B * H * n_blocks, T * D)
    chunks = [codec.pack_blocks(x, args.right, args.nbits, T)[0] for x in xs]
    p = sum(c.n_escapes for c in chunks) / (2 * n)
    jobs = (_lib.PackJob * 2)()
    keep = []
    for jb, x, c in zip(jobs, xs, chunks):
        meta = torch.zeros(n_blocks + 2, dtype=torch.int64, device=dev)
        esc = torch.empty(max(c.n_escapes, 16), dtype=torch.uint8, device=dev)
        hist = torch.zeros(256, dtype=torch.int32, device=dev)
        keep += [meta, esc, hist]
        sb, sh, ss, _ = x.stride()
        jb.src_bf16, jb.stride_b, jb.stride_h, jb.stride_s = x.data_ptr(), sb, sh, ss
        jb.n_blocks, jb.right = n_blocks, args.right
        jb.sign_mant, jb.codes, jb.escapes = c.sign_mant.data_ptr(), c.codes.data_ptr(), esc.data_ptr()
        jb.escapes_capacity = esc.numel()
        jb.tile_base, jb.seg_escape_offsets = c.tile_base.data_ptr(), meta.data_ptr()
        jb.hist256 = 0 if args.no_hist else hist.data_ptr()
    status = torch.zeros(2, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    outs = [torch.empty_like(x) for x in xs]
    tables = [codec.build_segment_table(c.segments(), None, dev) for c in chunks]
    todo = [(c.segments(), o, t) for c, o, t in zip(chunks, outs, tables)]

    def pack():
        _lib.check(L.adacode_pack_jobs(ctypes.addressof(jobs), 2, B, H, T, D, args.nbits, ws.data_ptr(), ws.numel(),
                                       status.data_ptr(), stream), 'adacode_pack_jobs')

    def unpack():
        codec.unpack_segments_multi(todo)

    t_pack = _time(pack, args.iters, args.warmup)
    t_unpack = _time(unpack, args.iters, args.warmup)
    assert int(status[0].item()) == 0
    for x, o in zip(xs, outs):
        assert torch.equal(o.view(torch.int16), x.view(torch.int16)), 'round trip is not bit-exact'
    alg = 2 * n * (3.0 + args.nbits / 8.0 + p)
    for name, t in (('pack_pair', t_pack), ('unpack_pair', t_unpack)):
        print(json.dumps({
            'kernel': name, 'shape': list(shape), 'nbits': args.nbits, 'right': args.right,
            'escape_fraction': round(p, 5), 'us': round(t * 1e6, 1),
            'algorithmic_GBps': round(alg / t / 1e9, 1), 'bf16_equiv_GBps': round(4 * n / t / 1e9, 1),
        }))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument('--shape', default='16,8,8192,128')
    ap.add_argument('--nbits', type=int, default=4)
    ap.add_argument('--right', type=int, default=131)
    ap.add_argument('--seq-tile', type=int, default=128)
    ap.add_argument('--iters', type=int, default=5)
    ap.add_argument('--warmup', type=int, default=2)
    ap.add_argument('--no-hist', action='store_true')
    ap.add_argument('--pair', action='store_true', help='a K and a V tensor per launch (job-table entry points)')
    ap.add_argument('--attention', type=int, default=0, metavar='HQ',
                    help='time decode attention with HQ query heads instead: fused (packed planes) '
                         'against unpack + torch SDPA over dense K/V')
    args = ap.parse_args()
    if args.attention:
        return attention_main(args)
    if args.pair:
        return pair_main(args)
    shape = tuple(int(v) for v in args.shape.split(','))
    B, H, S, D = shape
    dev = torch.device('cuda', 0)
    x = synthetic_keys(shape, device=dev)
    n = x.numel()
    T = args.seq_tile
    n_blocks = S // T
    chunk, _ = codec.pack_blocks(x, args.right, args.nbits, T, need_hist=True)
    p = chunk.n_escapes / n
    out = torch.empty_like(x)
    L = _lib.lib()
    sc = codec._scratch_for(dev)
    ws = sc.workspace_for(B * H * n_blocks, T * D)
    meta = torch.zeros(n_blocks + 2, dtype=torch.int64, device=dev)
    esc = torch.empty(max(chunk.n_escapes, 16), dtype=torch.uint8, device=dev)
    hist = torch.zeros(256, dtype=torch.int32, device=dev)
    sb, sh, ss, _ = x.stride()
    stream = torch.cuda.current_stream(dev).cuda_stream

    def pack():
        rc = L.adacode_pack_tiles(x.data_ptr(), sb, sh, ss, B, H, n_blocks, T, D, args.right, args.nbits,
                                  chunk.sign_mant.data_ptr(), chunk.codes.data_ptr(), esc.data_ptr(), esc.numel(),
                                  chunk.tile_base.data_ptr(), meta.data_ptr(),
                                  0 if args.no_hist else hist.data_ptr(), ws.data_ptr(), ws.numel(),
                                  meta.data_ptr() + 8 * (n_blocks + 1), stream)
        _lib.check(rc, 'adacode_pack_tiles')

    def unpack():
        codec.unpack_chunk(chunk, out)

    t_pack = _time(pack, args.iters, args.warmup)
    t_unpack = _time(unpack, args.iters, args.warmup)
    assert torch.equal(out.view(torch.int16), x.view(torch.int16)), 'round trip is not bit-exact'
    alg = n * (3.0 + args.nbits / 8.0 + p)
    for name, t in (('pack', t_pack), ('unpack', t_unpack)):
        print(json.dumps({
            'kernel': name, 'shape': list(shape), 'nbits': args.nbits, 'right': args.right,
            'escape_fraction': round(p, 5), 'us': round(t * 1e6, 1),
            'algorithmic_GBps': round(alg / t / 1e9, 1), 'bf16_equiv_GBps': round(2 * n / t / 1e9, 1),
        }))


if __name__ == '__main__':
    main()

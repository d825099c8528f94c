"""TEST HELPER: the codec interface of ``adacode_b200.codec`` served by the CPU oracle.

The cache classes reach the kernels through the module attribute ``codec`` of
``adacode_b200.float_cache_utils`` / ``mla_float_cache_utils``.  CPU tests swap that attribute
for this module (``monkeypatch.setattr``) so the host logic — the adjuster state machine —
can be replayed without a GPU.  The shipped package never imports this file.
"""
from __future__ import annotations

import numpy as np
import torch

from adacode_b200.codec import PackedChunk, TiledCompressedTensor  # plain containers
from oracle import float11_oracle as O


def pack_blocks(x, right, nbits, seq_tile=128, need_hist=False, hist_out=None, escape_capacity=None):
    if nbits not in (1, 2, 3, 4):
        raise ValueError(f'Tiled compressed path supports nbits in (1, 2, 3, 4), got {nbits}')
    x = x.to(torch.bfloat16)
    B, H, S, D = x.shape
    if S % seq_tile:
        raise ValueError('sequence length is not a multiple of seq_tile_size')
    n_blocks = S // seq_tile
    signs, codes, escs, bases, offs = [], [], [], [], [0]
    hist = np.zeros(256, np.int64)
    left = right - 2 ** nbits + 1
    for j in range(n_blocks):
        p = O.pack_block(x[:, :, j * seq_tile:(j + 1) * seq_tile].contiguous(), right, nbits, need_hist=need_hist)
        signs.append(p.sign_mass_data)
        codes.append(p.exp_data)
        escs.append(p.invalid_exp)
        bases.append(p.tile_invalid_base)
        offs.append(offs[-1] + p.invalid_exp.size)
        if need_hist:
            hist += p.hist
    chunk = PackedChunk(
        torch.from_numpy(np.stack(signs)), torch.from_numpy(np.stack(codes)),
        torch.from_numpy(np.concatenate(escs) if escs else np.zeros(0, np.uint8)),
        torch.from_numpy(np.stack(bases)), offs, torch.tensor(offs, dtype=torch.int64),
        left, int(right), int(nbits), B, H, seq_tile, D)
    h = None
    if need_hist:
        h = torch.from_numpy(hist).to(torch.int32)
        if hist_out is not None:
            hist_out += h
            h = hist_out
    return chunk, h


def _unpack_one(seg: TiledCompressedTensor) -> torch.Tensor:
    B, H, S, D = seg.original_shape
    p = O.PackedBlock(seg.sign_mass_data.contiguous().numpy(), seg.exp_data.contiguous().numpy(),
                      seg.invalid_exp.contiguous().numpy(), seg.tile_invalid_base.contiguous().numpy(),
                      int(seg.left), int(seg.right), int(seg.nbits), (B, H, S, D))
    return torch.from_numpy(O.unpack_block(p).view(np.int16)).view(torch.bfloat16).view(B, H, S, D)


def build_segment_table(segments, seq_offsets=None, device=None):
    offs, run = [], 0
    for i, seg in enumerate(segments):
        off = run if seq_offsets is None else int(seq_offsets[i])
        offs.append(off)
        run = off + int(seg.original_shape[-2])
    return torch.tensor(offs, dtype=torch.int64)


def unpack_segments(segments, dst, seq_offsets=None, table=None):
    if table is not None:
        seq_offsets = [int(v) for v in table.tolist()]
    run = 0
    for i, seg in enumerate(segments):
        off = run if seq_offsets is None else int(seq_offsets[i])
        T = int(seg.original_shape[-2])
        dst[:, :, off:off + T].copy_(_unpack_one(seg))
        run = off + T


def unpack_segments_multi(jobs):
    for segments, dst, table in jobs:
        if segments:
            unpack_segments(segments, dst, table=table)


def exponent_hist(x, hist_out=None):
    h = torch.from_numpy(O.exponent_hist(x.to(torch.bfloat16).contiguous())).to(torch.int32)
    if hist_out is not None:
        hist_out += h
        return hist_out
    return h


def analysis_best_bits(data_freq, store_index=False):
    return O.choose_params(np.asarray(data_freq.tolist() if hasattr(data_freq, 'tolist') else data_freq, np.int64))


def pack_pair(k, v, k_params, v_params, seq_tile=128, need_hist=False, capacities=(None, None)):
    k_chunk, k_hist = pack_blocks(k, k_params[0], k_params[1], seq_tile, need_hist)
    v_chunk, v_hist = pack_blocks(v, v_params[0], v_params[1], seq_tile, need_hist)
    kh = k_hist.numpy().copy() if need_hist else None
    vh = v_hist.numpy().copy() if need_hist else None
    return k_chunk, v_chunk, k_hist, v_hist, kh, vh


def read_back(t):
    return t.cpu().numpy()

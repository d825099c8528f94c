"""Sharding one logical float11 cache over several GPUs (one process per GPU).

Every (batch, kv head, block) tile is packed independently, so batch sequences (or KV heads)
are simply dealt out to ranks and each rank keeps its own ``Float11Cache``.  Two things tie
the shards together:

* the code-length adjuster must see the exponent histogram of the WHOLE batch, so that every
  shard adopts the window the unsharded cache would adopt: ``HistogramAllReduce`` is passed to
  the cache as ``hist_reduce`` and sums the int32[256] histograms over the process group
  (NCCL on GPUs, gloo in CPU tests).  This is the only collective of the path and it runs on
  adjust steps only;
* the canonical byte stream of a block of the whole batch is the concatenation of the shards'
  streams in rank order: ``merge_shard_segments`` rebuilds it (escape lists appended, tile
  bases of later shards shifted by the escape totals before them), which is what parity
  against the unsharded reference is checked on.

The reference has no multi-GPU path; its segment layout ([b][h]-major planes, one escape list
per block with inclusive per-tile counts — compress_tiled_kv.py:524-588) is what makes the
concatenation rule exact.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist


def shard_range(n_items: int, world_size: int, rank: int) -> range:
    """Contiguous share of ``n_items`` (sequences or heads) for ``rank``; earlier ranks take the
    remainder."""
    base, extra = divmod(int(n_items), int(world_size))
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


class HistogramAllReduce:
    """Callable ``hist -> hist summed over the group`` for ``Float11Cache(hist_reduce=...)``.
    Every rank must update its layers in the same order (it does: same model, same step)."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.calls = 0

    def __call__(self, hist: torch.Tensor) -> torch.Tensor:
        if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(self.group) == 1:
            return hist
        out = hist.to(torch.int32).clone()
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.group)
        self.calls += 1
        return out


def merge_shard_segments(states: Sequence[dict], dim: str = 'batch') -> dict:
    """One exported segment state per rank (same block, same window) -> the state of the whole
    batch.  ``dim='batch'`` when sequences were sharded; heads cannot be merged by plain
    concatenation (planes are [b][h]-major) unless batch is 1, which ``dim='head'`` requires."""
    first = states[0]
    for st in states[1:]:
        if (st['right'], st['nbits']) != (first['right'], first['nbits']):
            raise ValueError('shards of one block must share window and code length')
    B0, H0, S, D = tuple(first['original_shape'])
    if dim == 'head' and any(tuple(st['original_shape'])[0] != 1 for st in states):
        raise ValueError("dim='head' needs batch size 1 per shard")
    bases, offset = [], 0
    for st in states:
        bases.append(st['tile_invalid_base'].to(torch.int64) + offset)
        offset += int(st['invalid_exp'].numel())
    merged = dict(first)
    merged['sign_mass_data'] = torch.cat([st['sign_mass_data'] for st in states])
    merged['exp_data'] = torch.cat([st['exp_data'] for st in states])
    merged['invalid_exp'] = torch.cat([st['invalid_exp'] for st in states])
    merged['tile_invalid_base'] = torch.cat(bases).to(torch.int32)
    if dim == 'batch':
        merged['original_shape'] = (sum(tuple(st['original_shape'])[0] for st in states), H0, S, D)
    else:
        heads = sum(tuple(st['original_shape'])[1] for st in states)
        merged['original_shape'] = (1, heads, S, D)
        merged['num_kv_heads'] = heads
    n = 1
    for d in merged['original_shape']:
        n *= d
    merged['n_elements'] = n
    return merged

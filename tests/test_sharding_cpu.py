"""Two gloo ranks on the CPU: each owns half of the batch (or half of the KV heads) of one
logical cache, histograms are all-reduced at adjust steps, and the concatenation of the two
shards' byte streams must be exactly what the reference produced for the unsharded cache."""
import json
import os
import socket
import warnings

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests import scenarios
from tests.test_state_machine_cpu import GOLDEN


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, name, dim, out_path):
    import adacode_b200.float_cache_utils as fc
    import adacode_b200.mla_float_cache_utils as mc
    from adacode_b200 import sharding
    from tests import oracle_codec
    fc.codec = oracle_codec
    mc.codec = oracle_codec
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        sc = scenarios.SCENARIOS[name]
        cfg = scenarios.StubConfig(sc.num_layers, **sc.config_extra)
        reducer = sharding.HistogramAllReduce()
        cache = fc.Float11Cache(cfg, hist_reduce=reducer, **sc.cache_kwargs)
        for per_layer in sc.steps():
            for l, (k, v) in enumerate(per_layer):
                n = k.shape[0] if dim == 'batch' else k.shape[1]
                mine = sharding.shard_range(n, world, rank)
                sl = slice(mine.start, mine.stop)
                ks, vs = (k[sl], v[sl]) if dim == 'batch' else (k[:, sl], v[:, sl])
                out_k, out_v = cache.update(ks, vs, l)
                assert out_k.shape[-2] == cache.get_seq_length(l)
        layer = cache.layers[0]
        mine = {'key': layer._compressed_prefix_key_segments, 'value': layer._compressed_prefix_value_segments,
                'params': [layer.keys_right, layer.keys_nbits, layer.values_right, layer.values_nbits],
                'updates': [layer.keys_update_times, layer.values_update_times], 'reduces': reducer.calls}
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        if rank == 0:
            result = {'params': gathered[0]['params'], 'updates': gathered[0]['updates'],
                      'same_params': all(g['params'] == gathered[0]['params'] for g in gathered),
                      'reduces': gathered[0]['reduces'], 'key_segments': [], 'value_segments': []}
            for side in ('key', 'value'):
                for j in range(len(gathered[0][side])):
                    merged = sharding.merge_shard_segments([g[side][j] for g in gathered], dim=dim)
                    result[f'{side}_segments'].append(scenarios.segment_digest(merged))
            json.dump(result, open(out_path, 'w'))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('name,dim', [('batch2_aligned', 'batch'), ('scale_shift_adjust', 'head')])
def test_two_shards_reproduce_the_unsharded_reference(tmp_path, name, dim):
    out = tmp_path / 'merged.json'
    with warnings.catch_warnings():
        warnings.simplefilter('ignore')
        mp.spawn(_worker, args=(2, _free_port(), name, dim, str(out)), nprocs=2, join=True)
    got = json.load(open(out))
    gold = GOLDEN[name]['layers'][0]
    assert got['same_params'] and got['params'] == gold['params']
    assert got['updates'] == [gold['memory']['keys_update_times'], gold['memory']['values_update_times']]
    assert got['reduces'] > 0
    assert got['key_segments'] == gold['key_segments']
    assert got['value_segments'] == gold['value_segments']


def test_shard_range_covers_everything():
    from adacode_b200.sharding import shard_range
    for n in (1, 7, 8, 64):
        for w in (1, 2, 3, 8):
            got = [i for r in range(w) for i in shard_range(n, w, r)]
            assert got == list(range(n))

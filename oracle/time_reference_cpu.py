"""TEST INFRASTRUCTURE, not part of the product: times the REFERENCE's own CPU-runnable pack on a
sample of the benchmark workload, where the reference source tree is available.

    python oracle/time_reference_cpu.py /path/to/reference [n_blocks]

The reference has no compiled code; its pure-torch pack (``compress_open_tiled_rows`` +
``seal_open_tiled_rows``, compress_tiled_kv.py:721-751, :633-718) needs no GPU and no Triton
interpreter and is byte-identical to its Triton pack.  It handles one sequence and one 128-token
block per call, so the sample is looped over sequences and blocks, as the reference's cache would.
Its only unpack is a Triton kernel; one block is decoded under ``TRITON_INTERPRET=1`` for the
record.  Prints one JSON line.
"""
from __future__ import annotations

import json
import os
import sys
import tempfile
import time

os.environ.setdefault('TRITON_INTERPRET', '1')
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit('usage: time_reference_cpu.py <reference checkout> [n_blocks]')
    tmp = tempfile.mkdtemp(prefix='refpkg_')
    os.symlink(os.path.abspath(sys.argv[1]), os.path.join(tmp, 'kv_compression'))
    sys.path.insert(0, tmp)
    n_blocks = int(sys.argv[2]) if len(sys.argv) > 2 else 32
    import torch
    from kv_compression import compress_tiled_kv as ref
    import bench
    calib = bench.s4_calibration(range(1))
    out = {'threads': torch.get_num_threads(), 'cpu_count': os.cpu_count(), 'blocks_per_tensor': n_blocks,
           'sample': f'layer 0, sequence 0 of the stress workload, first {n_blocks} 128-token blocks of K and V '
                     '[1,8,128,128] each'}
    total_s, elems = 0.0, 0
    sealed = None
    for which in ('k', 'v'):
        right, nbits = calib[(0, which)]
        x = bench.s4_slab(0, which, 0, 1, 0, n_blocks * 128, 'cpu', window=(right, nbits))
        ref.seal_open_tiled_rows(ref.compress_open_tiled_rows(x[:, :, :128].contiguous(), right=right, nbits=nbits)[0])
        t0 = time.perf_counter()
        for j in range(n_blocks):
            blk = x[:, :, j * 128:(j + 1) * 128].contiguous()
            rows, _hist = ref.compress_open_tiled_rows(blk, right=right, nbits=nbits, need_adjust=True)
            sealed = ref.seal_open_tiled_rows(rows)
        total_s += time.perf_counter() - t0
        elems += x.numel()
    out['pure_torch_pack_bf16_equiv_GBps'] = round(2 * elems / total_s / 1e9, 4)
    out['pure_torch_pack_ms_per_block'] = round(total_s * 1e3 / (2 * n_blocks), 3)
    t0 = time.perf_counter()
    back = sealed.materialize()
    dt = time.perf_counter() - t0
    out['triton_interpreter_unpack_ms_per_block'] = round(dt * 1e3, 1)
    out['triton_interpreter_unpack_bf16_equiv_GBps'] = round(2 * back.numel() / dt / 1e9, 5)
    print(json.dumps(out))


if __name__ == '__main__':
    main()

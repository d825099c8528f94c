"""Model weights kept packed and decoded just in time, on the flat float11 codec.

Interface of the reference's ``manager.py``: ``convert_model(model, model_config, is_tie_weight,
release_hook)`` (:81-159) replaces the listed parameters of every configured block by one packed
buffer (``CompressorBitMap``), registers a forward pre-hook on the block's ``decode_hook_name``
module that decodes the buffer and hands each child module a view of it as its ``weight`` /
``bias``, and a forward hook on ``release_hook_name`` that drops those views again
(``get_decode_hook`` :46-72, ``get_release_hook`` :75-79); ``get_mem_pool_info`` (:13-44) reports the
largest configured weight.

``model_config`` maps block ids to
``{'model_names', 'decode_hook_name', 'release_hook_name', 'model_shapes', 'model_n_elements',
'best_indices' (last entry = right edge of the window), 'nbits'}``; ``build_block_config`` derives
such a mapping from a model (the reference reads it from a JSON its analysis scripts write).

One deliberate difference: the reference's decode hook forgets the packed planes after its first
run (:71, "only prefill compression"), which leaves later forwards without weights once the
release hook has dropped the views.  Here the planes stay, every forward decodes into a buffer
shared by all blocks of a device (sized for the largest block), and the release hook only drops
the views.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import codec
from .compress_bitmap_merge import CompressorBitMap


def _split_name(weight_name: str):
    parent, _, leaf = weight_name.rpartition('.')
    if leaf not in ('weight', 'bias'):
        raise AssertionError('must be weight or bias')
    return parent, leaf


def get_mem_pool_info(model_config, model: torch.nn.Module) -> dict:
    """Largest weight among ``(weight_name, nbit, right)`` entries (reference: :13-44)."""
    best_name, best_numel = None, 0
    for weight_name, _nbit, _right in model_config:
        parts = weight_name.split('.')
        if parts[-1] in ('weight', 'bias'):
            parts = parts[:-1]
        module = model if 'lm_head' in weight_name and len(parts) == 1 else model.get_submodule('.'.join(parts))
        numel = module.weight.numel()
        if numel > best_numel:
            best_name, best_numel = weight_name, numel
    return {'max_numel': best_numel, 'max_weight_name': best_name}


class _DecodePool:
    """One dense bf16 buffer per device, as large as the largest packed block registered on it."""

    def __init__(self):
        self.buffers: dict = {}
        self.need: dict = {}

    def reserve(self, device, numel: int) -> None:
        self.need[device] = max(self.need.get(device, 0), int(numel))

    def get(self, device, numel: int) -> torch.Tensor:
        buf = self.buffers.get(device)
        if buf is None or buf.numel() < numel:
            buf = self.buffers[device] = torch.empty(max(self.need.get(device, 0), numel), dtype=torch.bfloat16,
                                                      device=device)
        return buf[:numel]


def get_decode_hook(block_id, pool: Optional[_DecodePool] = None):
    """Forward pre-hook: decode the module's packed block and install the parameter views."""
    def decode_hook(module, _inputs):
        comp = module.compressor
        if comp.device is None:
            return
        n = comp.n_elements
        dense = pool.get(comp.device, n) if pool is not None else torch.empty(n, dtype=torch.bfloat16, device=comp.device)
        comp.uncompress_with_weights(dense)
        for child, shape, part, piece in zip(module.childen, module.model_shapes, module.module_part,
                                             torch.tensor_split(dense, module.split_positions)):
            child.__dict__[part] = piece.view(shape)
    return decode_hook


def get_release_hook(block_id):
    """Forward hook: drop the parameter views installed by the decode hook."""
    def release_hook(module, _inputs, _output):
        for child, part in zip(module.childen, module.module_part):
            child.__dict__.pop(part, None)
    return release_hook


def _split_positions(sizes):
    out, run = [], 0
    for n in sizes[:-1]:
        run += int(n)
        out.append(run)
    return out


def convert_model(model, model_config, is_tie_weight: bool = True, release_hook: bool = True):
    """Pack the configured parameters and register the hooks (reference: :81-159)."""
    pool = _DecodePool()
    model._float11_weight_pool = pool
    packed_first = None
    for block_id, spec in model_config.items():
        owners, parts, flats = [], [], []
        for name in spec['model_names']:
            parent, leaf = _split_name(name)
            owner = model.get_submodule(parent)
            flats.append(getattr(owner, leaf).data.detach().to(torch.bfloat16).reshape(-1).clone())
            delattr(owner, leaf)
            owners.append(owner)
            parts.append(leaf)
        sizes = spec['model_n_elements']
        assert len(spec['model_shapes']) == len(sizes), f'{block_id=}'
        comp = CompressorBitMap(spec['best_indices'][-1], spec['nbits'])
        comp.compress(torch.cat(flats))
        pool.reserve(comp.device, comp.n_elements)
        host = model.get_submodule(spec['decode_hook_name'])
        host.register_forward_pre_hook(get_decode_hook(block_id, pool))
        host.model_shapes = spec['model_shapes']
        host.split_positions = _split_positions(sizes)
        host.compressor = comp
        host.childen = owners              # (the reference's attribute name)
        host.module_part = parts
        if release_hook:
            tail = model.get_submodule(spec['release_hook_name'])
            tail.childen = owners
            tail.module_part = parts
            tail.register_forward_hook(get_release_hook(block_id))
        if block_id == 0 or str(block_id) == '0':
            packed_first = (comp, spec)
    if is_tie_weight:
        # the output projection shares block 0 (the embedding): decode it again where it is used
        if packed_first is None:
            raise KeyError('is_tie_weight needs block 0 (the embedding) in model_config')
        comp, spec = packed_first
        head = model.lm_head
        if 'weight' in head._parameters:
            delattr(head, 'weight')
        head.register_forward_pre_hook(get_decode_hook(0, pool))
        head.model_shapes = spec['model_shapes']
        head.split_positions = _split_positions(spec['model_n_elements'])
        head.compressor = comp
        head.childen = [head]
        head.module_part = ['weight']
        if release_hook:
            head.register_forward_hook(get_release_hook(0))
    return model


def build_block_config(model, blocks: dict) -> dict:
    """``model_config`` for ``convert_model``: ``blocks`` maps a block id to
    ``(decode_hook_name, release_hook_name, [parameter names])``; window and code length of a block
    come from the exponent histogram of its parameters by the run-time adjuster's rule."""
    config = {}
    for block_id, (decode_name, release_name, names) in blocks.items():
        shapes, sizes = [], []
        hist = None
        for name in names:
            parent, leaf = _split_name(name)
            p = getattr(model.get_submodule(parent), leaf).data
            shapes.append(tuple(p.shape))
            sizes.append(p.numel())
            flat = p.detach().to(torch.bfloat16).reshape(1, 1, -1, 8)
            hist = codec.exponent_hist(flat, hist_out=hist)
        right, nbits = codec.analysis_best_bits(codec.read_back(hist))
        config[block_id] = {'model_names': list(names), 'decode_hook_name': decode_name, 'release_hook_name': release_name,
                            'model_shapes': shapes, 'model_n_elements': sizes, 'best_indices': [right], 'nbits': nbits}
    return config

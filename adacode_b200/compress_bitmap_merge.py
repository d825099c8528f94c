"""Flat float11 codec: ``CompressorBitMap`` with the interface of the reference's
``compress_bitmap_merge.py`` (:633-873), served by the sm_100a kernels.

The flat layout packs ANY bf16 tensor (KV blocks of the 'legacy' cache layout, model weights) as
one sign/mantissa byte per element, n-bit exponent codes, one compact list of escaped exponents
in flat order and ``block_base``: the inclusive running escape count per ``invalid_block_size``
(= 128 x {8, 4, 8, 2}[nbits - 1]) elements.  These are exactly the planes ``adacode_pack_tiles``
writes for tiles of one block each, so ``compress`` is one such launch; ``uncompress`` goes
through ``adacode_unpack_flat``, which decodes 16384-element tiles and takes every
(16384 / block)-th base.  There is no CPU path.
"""
from __future__ import annotations

import torch

from . import _lib, codec

_BLOCK_GAPS = (8, 4, 8, 2)
_MAX_ELEMS_PER_CALL = 1 << 30


def _ones_code_bytes(nbits: int, n_bytes: int, device) -> torch.Tensor:
    """Code bytes in which every code is 1 (an in-window code): padding that needs no escape."""
    pattern = {1: [0xFF], 2: [0x55], 3: [0x24, 0x92, 0x49], 4: [0x11]}[nbits]
    reps = (n_bytes + len(pattern) - 1) // len(pattern)
    return torch.tensor(pattern * reps, dtype=torch.uint8, device=device)[:n_bytes]


class CompressorBitMap:
    """reference: compress_bitmap_merge.py:633-873."""

    def __init__(self, right=129, nbits=3):
        self.device = None
        self.original_shape = None
        self.n_elements = None
        self.n_exp_data = None
        self.sign_mass_data = None
        self.exp_data = None
        self.invalid_exp = None
        self.blocksize = 128
        self.left = right - 2 ** nbits + 1
        self.right = right
        self.nbits = nbits
        self._configure_runtime()
        self.block_base = None          # int64, as the reference's torch.cumsum yields it
        self._base_i32 = None           # the same counts as the kernels read them

    def _configure_runtime(self):
        if self.nbits not in (1, 2, 3, 4):
            raise IndexError('list index out of range')          # the reference indexes a 4-entry list
        self.invalid_block_size = self.blocksize * _BLOCK_GAPS[self.nbits - 1]
        self.left_nbits = self.left << 7

    def reset_memory(self):
        self.device = None
        self.n_elements = None
        self.n_exp_data = None
        self.original_shape = None
        self.sign_mass_data = None
        self.exp_data = None
        self.invalid_exp = None
        self.block_base = None
        self._base_i32 = None

    def _update_compression_params(self, right, nbits):
        self.left = right - 2 ** nbits + 1
        self.right = right
        self.nbits = nbits
        self._configure_runtime()
        self.block_base = None

    def get_memory(self):
        if self.sign_mass_data is None:
            return {'compressed_memory': 0, 'original_memory': 0}
        compressed = (self.sign_mass_data.numel() + self.exp_data.numel()
                      + (0 if self.invalid_exp is None else self.invalid_exp.numel())
                      + (0 if self.block_base is None else self.block_base.numel() * self.block_base.element_size()))
        original = 0 if self.n_elements is None else self.n_elements * 2
        return {'compressed_memory': compressed, 'original_memory': original,
                'ratio': 0 if original == 0 else compressed / original}

    _STATE_KEYS = ('right', 'nbits', 'left', 'left_nbits', 'blocksize', 'invalid_block_size', 'device',
                   'original_shape', 'n_elements', 'n_exp_data', 'sign_mass_data', 'exp_data', 'invalid_exp',
                   'block_base')

    def export_state(self):
        return {k: getattr(self, k) for k in self._STATE_KEYS}

    def export_decode_view(self):
        return self.export_decode_view_from_state(self.export_state())

    @staticmethod
    def export_decode_view_from_state(state):
        keys = ('sign_mass_data', 'exp_data', 'invalid_exp', 'block_base', 'left', 'right', 'left_nbits', 'nbits',
                'blocksize', 'invalid_block_size', 'original_shape', 'n_elements', 'n_exp_data', 'device')
        return {k: state[k] for k in keys}

    @classmethod
    def from_state(cls, state):
        c = cls(right=state['right'], nbits=state['nbits'])
        for k in ('device', 'original_shape', 'n_elements', 'n_exp_data', 'sign_mass_data', 'exp_data',
                  'invalid_exp', 'block_base'):
            setattr(c, k, state[k])
        return c

    @classmethod
    def compress_block(cls, original_data_bfloat16, right, nbits, need_adjust=False):
        c = cls(right=right, nbits=nbits)
        hist = c.compress(original_data_bfloat16, need_adjust=need_adjust)
        return c, hist

    def materialize(self):
        return self.uncompress()

    # ------------------------------------------------------------------ pack
    def compress(self, original_data_bfloat16, need_adjust=False):
        """Pack the tensor (any shape, bf16, element count a multiple of 8); returns the int32[256]
        exponent histogram when ``need_adjust`` (reference: :768-822, :210-254)."""
        x = original_data_bfloat16
        if x.dtype != torch.bfloat16:
            raise ValueError(f'expected a bfloat16 tensor, got {x.dtype}')
        self.device = x.device
        self.original_shape = x.shape
        n = self.n_elements = x.numel()
        assert n % 8 == 0, 'the packed code plane holds whole groups of 8 elements'
        ibs = self.invalid_block_size
        flat = x.reshape(-1)
        if not flat.is_contiguous():
            flat = flat.contiguous()
        n_blocks = (n + ibs - 1) // ibs
        n_pad = n_blocks * ibs
        real_tail_escapes = None
        if n_pad != n:
            # whole blocks only: pad with zeros (they escape, after every real element of the last
            # block) and drop their escape bytes again below
            tail = flat[(n_blocks - 1) * ibs:]
            e = (tail.view(torch.int16).to(torch.int32) >> 7) & 0xFF
            real_tail_escapes = int(((e <= self.left) | (e > self.right)).sum().item())
            flat = torch.cat([flat, torch.zeros(n_pad - n, dtype=torch.bfloat16, device=x.device)])
        hist = torch.zeros(256, dtype=torch.int32, device=x.device) if need_adjust else None
        per_call = max(ibs, (_MAX_ELEMS_PER_CALL // ibs) * ibs)
        signs, codes, escs, bases = [], [], [], []
        carried = 0
        for lo in range(0, n_pad, per_call):
            hi = min(n_pad, lo + per_call)
            part = flat[lo:hi].view(1, (hi - lo) // ibs, ibs // 32, 32)
            chunk, _ = codec.pack_blocks(part, self.right, self.nbits, ibs // 32, need_hist=need_adjust, hist_out=hist)
            signs.append(chunk.sign_mant.reshape(-1))
            codes.append(chunk.codes.reshape(-1))
            escs.append(chunk.escapes)
            bases.append(chunk.tile_base.reshape(-1) + carried if carried else chunk.tile_base.reshape(-1))
            carried += chunk.n_escapes
        self.sign_mass_data = signs[0] if len(signs) == 1 else torch.cat(signs)
        self.exp_data = codes[0] if len(codes) == 1 else torch.cat(codes)
        self.invalid_exp = escs[0] if len(escs) == 1 else torch.cat(escs)
        base = (bases[0] if len(bases) == 1 else torch.cat(bases)).to(torch.int32)
        if n_pad != n:
            pad = n_pad - n
            before_last = int(base[-2].item()) if n_blocks > 1 else 0
            keep = before_last + real_tail_escapes
            self.invalid_exp = self.invalid_exp[:keep].clone()
            base = base.clone()
            base[-1] = keep
            self.sign_mass_data = self.sign_mass_data[:n].clone()
            self.exp_data = self.exp_data[: n * self.nbits // 8].clone()
            if hist is not None:
                hist[0] -= pad                       # the padding's exponent is 0
        self._base_i32 = base
        self.block_base = base.to(torch.int64)
        self.n_exp_data = n * self.nbits // 8
        return hist

    def _kernel_base(self) -> torch.Tensor:
        if self._base_i32 is None or self._base_i32.numel() != self.block_base.numel():
            self._base_i32 = self.block_base.to(torch.int32).contiguous()
        return self._base_i32

    # ------------------------------------------------------------------ unpack
    def uncompress_with_weights(self, uncompressed_odb):
        """Decode into ``uncompressed_odb`` (a flat 16-bit view of ``n_elements`` elements, bf16 or
        uint16/int16 storage; reference: :872-873)."""
        out = uncompressed_odb
        if out.numel() != self.n_elements or out.element_size() != 2 or not out.is_contiguous():
            raise ValueError('uncompress_with_weights needs a contiguous 16-bit buffer of n_elements elements')
        n, ibs = self.n_elements, self.invalid_block_size
        n_whole = (n // ibs) * ibs
        dev = self.device
        sc = codec._scratch_for(dev)
        esc = self.invalid_exp
        stream = codec._stream_ptr(dev)
        L = _lib.lib()
        with torch.cuda.device(dev):
            if n_whole:
                rc = L.adacode_unpack_flat(self.sign_mass_data.data_ptr(), self.exp_data.data_ptr(),
                                           esc.data_ptr() if esc.numel() else 0, esc.numel(),
                                           self._kernel_base().data_ptr(), n_whole, self.left, self.nbits,
                                           out.data_ptr(), sc.status.data_ptr(), stream)
                _lib.check(rc, 'adacode_unpack_flat')
            if n_whole != n:
                # ragged last block: decode a padded copy of its planes (padding codes are in-window)
                r = n - n_whole
                sm = torch.zeros(ibs, dtype=torch.uint8, device=dev)
                sm[:r] = self.sign_mass_data[n_whole:]
                cd = _ones_code_bytes(self.nbits, ibs * self.nbits // 8, dev).clone()
                cd[: r * self.nbits // 8] = self.exp_data[n_whole * self.nbits // 8:]
                prev = int(self.block_base[-2].item()) if self.block_base.numel() > 1 else 0
                tail_esc = esc[prev:].contiguous()
                base = torch.tensor([tail_esc.numel()], dtype=torch.int32, device=dev)
                tmp = torch.empty(ibs, dtype=torch.int16, device=dev)
                rc = L.adacode_unpack_flat(sm.data_ptr(), cd.data_ptr(), tail_esc.data_ptr() if tail_esc.numel() else 0,
                                           tail_esc.numel(), base.data_ptr(), ibs, self.left, self.nbits,
                                           tmp.data_ptr(), sc.status.data_ptr(), stream)
                _lib.check(rc, 'adacode_unpack_flat')
                out.view(torch.int16)[n_whole:] = tmp[:r]

    def uncompress(self):
        out = torch.empty(self.n_elements, dtype=torch.bfloat16, device=self.device)
        self.uncompress_with_weights(out)
        return out.view(self.original_shape)

    def update_compress(self, right, nbits):
        """Decode, forget the planes and adopt a new window (reference: :846-864)."""
        dense = self.uncompress()
        self.reset_memory()
        self._update_compression_params(right, nbits)
        return dense

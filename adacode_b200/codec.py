"""Tiled float11 codec: torch-facing wrappers over the sm_100a kernels.

Mirrors the interface of the reference's ``compress_tiled_kv.py`` (``compress_tiled_tensor``,
``TiledCompressedTensor``, ``materialize_tiled_state``) and adds the batched forms the cache
uses: one launch packs every 128-token block of a prefill (``pack_blocks``), one launch
unpacks any list of segments (``unpack_segments``).

All tensors are CUDA tensors; kernels run on ``torch.cuda.current_stream``.  There is no CPU
path: on a CPU tensor, or without the built library, these functions raise.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Any, Optional, Sequence

import torch

from . import _lib

_SUPPORTED_TILE_NBITS = (1, 2, 3, 4)
_DEFAULT_TILE_NBITS = 3


# --------------------------------------------------------------------------------------
# per-device scratch
# --------------------------------------------------------------------------------------

class _DeviceScratch:
    """Pack scratch and the device status word of one GPU (grown on demand, reused)."""

    def __init__(self, device: torch.device):
        self.device = device
        self.workspace = torch.zeros(1 << 20, dtype=torch.uint8, device=device)
        self.status = torch.zeros(2, dtype=torch.int32, device=device)
        self.mailbox: Optional[torch.Tensor] = None      # pinned host bytes that kernels write results into
        self.mail_event = torch.cuda.Event()

    def workspace_for(self, n_tiles: int, tile_elems: int) -> torch.Tensor:
        need = int(_lib.lib().adacode_pack_workspace_bytes(n_tiles, tile_elems))
        if self.workspace.numel() < need:
            # the library wants a zero-filled scratch and leaves it reusable
            self.workspace = torch.zeros(int(need * 1.25) + 256, dtype=torch.uint8, device=self.device)
        return self.workspace


_scratch: dict[torch.device, _DeviceScratch] = {}


def _scratch_for(device: torch.device) -> _DeviceScratch:
    device = torch.device(device)
    if device.type != 'cuda':
        raise _lib.AdacodeError(f'float11 kernels need a CUDA tensor, got device {device} (there is no CPU path)')
    if device.index is None:
        device = torch.device('cuda', torch.cuda.current_device())
    s = _scratch.get(device)
    if s is None:
        s = _scratch[device] = _DeviceScratch(device)
    return s


def _stream_ptr(device: torch.device) -> int:
    return int(torch.cuda.current_stream(device).cuda_stream)


def read_back(t: torch.Tensor):
    """Host copy (numpy array of ``t``'s shape and dtype) of a small device tensor.

    The reference reads such values with ``.to('cpu')`` / ``.item()`` (escape totals,
    compress_tiled_kv.py:559-588; histograms, float_cache_utils.py:373), i.e. with cudaMemcpy, which
    queues behind whatever bulk transfer occupies the copy engine.  Here a one-CTA kernel stores the
    bytes into pinned host memory (``adacode_copy_to_host``) and the host waits for an event."""
    if not t.is_contiguous():
        t = t.contiguous()
    nbytes = t.numel() * t.element_size()
    if nbytes == 0 or nbytes % 4 != 0 or nbytes > (1 << 20):
        return t.cpu().numpy()
    dev = t.device
    sc = _scratch_for(dev)
    if sc.mailbox is None or sc.mailbox.numel() < nbytes:
        sc.mailbox = torch.empty(max(1 << 16, nbytes), dtype=torch.uint8).pin_memory()
    stream = torch.cuda.current_stream(dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().adacode_copy_to_host(t.data_ptr(), sc.mailbox.data_ptr(), nbytes, int(stream.cuda_stream))
    if rc == _lib.ERR_INVALID_ARG:
        return t.cpu().numpy()           # pinned memory this device cannot address: plain copy
    _lib.check(rc, 'adacode_copy_to_host')
    sc.mail_event.record(stream)
    sc.mail_event.synchronize()
    import numpy as np
    out = sc.mailbox[:nbytes].numpy().copy()
    return out.view(np.dtype(str(t.dtype).replace('torch.', ''))).reshape(tuple(t.shape))


def check_device_status(device) -> None:
    """Read the device status word (synchronises) and raise if a kernel flagged a problem."""
    s = _scratch_for(torch.device(device))
    word = int(read_back(s.status)[0])
    if word:
        s.status.zero_()
        raise _lib.AdacodeError('device status: ' + describe_status(word))


_STATUS_TEXT = (
    (_lib.STATUS_ESCAPE_OVERFLOW, 'escape buffer too small during pack'),
    (_lib.STATUS_ESCAPE_UNDERRUN, 'escape list shorter than the code plane requires during unpack'),
    (_lib.STATUS_TIMEOUT, 'a bounded on-chip wait gave up (results of that launch are invalid)'),
    (_lib.STATUS_MISALIGNED, 'a plane pointer in a segment record is not 16-byte aligned (tile skipped)'),
)


def describe_status(word: int) -> str:
    """Text for the bits of a device status word (every bit is named; unknown bits are shown in hex)."""
    parts = [text for bit, text in _STATUS_TEXT if word & bit]
    rest = word & ~sum(bit for bit, _ in _STATUS_TEXT)
    if rest:
        parts.append(f'unknown status bits {rest:#x}')
    return '; '.join(parts) if parts else 'ok'


# --------------------------------------------------------------------------------------
# containers
# --------------------------------------------------------------------------------------

@dataclass
class TiledCompressedTensor:
    """One packed block, field for field the reference's dataclass
    (compress_tiled_kv.py:238-342)."""

    sign_mass_data: torch.Tensor
    exp_data: torch.Tensor
    invalid_exp: torch.Tensor
    tile_invalid_base: torch.Tensor
    left: int
    right: int
    nbits: int
    original_shape: tuple
    seq_tile_size: int
    head_dim: int
    tile_head_dim: int
    tile_num_lanes: int
    num_sequence_tiles: int
    num_kv_heads: int
    device: torch.device
    layout: str = 'tiled'
    decode_kind: str = 'tiled_decode'
    has_outliers: bool = True

    @property
    def n_elements(self) -> int:
        n = 1 if self.original_shape else 0
        for d in self.original_shape:
            n *= d
        return n

    def get_memory(self) -> dict:
        """compress_tiled_kv.py:269-282."""
        compressed = (self.sign_mass_data.numel() + self.exp_data.numel() + self.invalid_exp.numel()
                      + self.tile_invalid_base.numel() * self.tile_invalid_base.element_size())
        original = self.n_elements * 2
        return {
            'compressed_memory': compressed,
            'original_memory': original,
            'ratio': 0.0 if original == 0 else compressed / original,
        }

    def export_state(self) -> dict:
        """compress_tiled_kv.py:284-306."""
        state = {
            'layout': self.layout, 'right': self.right, 'nbits': self.nbits, 'left': self.left,
            'device': self.device, 'original_shape': self.original_shape,
            'sign_mass_data': self.sign_mass_data, 'exp_data': self.exp_data,
            'seq_tile_size': self.seq_tile_size, 'head_dim': self.head_dim,
            'tile_head_dim': self.tile_head_dim, 'tile_num_lanes': self.tile_num_lanes,
            'num_sequence_tiles': self.num_sequence_tiles, 'num_kv_heads': self.num_kv_heads,
            'n_elements': self.n_elements, 'has_outliers': self.has_outliers,
        }
        if self.has_outliers:
            state['invalid_exp'] = self.invalid_exp
            state['tile_invalid_base'] = self.tile_invalid_base
        return state

    def export_decode_view(self) -> dict:
        state = self.export_state()
        state['kind'] = self.decode_kind
        return state

    def materialize(self) -> torch.Tensor:
        """compress_tiled_kv.py:313-337."""
        B, H, S, D = self.original_shape
        out = torch.empty((B, H, S, D), dtype=torch.bfloat16, device=self.sign_mass_data.device)
        unpack_segments([self], out)
        return out


class SegmentRef:
    """Handle on segment ``j`` of a ``PackedChunk``: everything the cache's bookkeeping needs
    (window, shape, escape count, byte accounting) is arithmetic on the chunk, so a prefill of
    hundreds of blocks creates no per-block tensor views; ``view()`` materialises the reference-
    shaped ``TiledCompressedTensor`` on demand."""

    __slots__ = ('chunk', 'j')

    def __init__(self, chunk: 'PackedChunk', j: int):
        self.chunk = chunk
        self.j = int(j)

    left = property(lambda self: self.chunk.left)
    right = property(lambda self: self.chunk.right)
    nbits = property(lambda self: self.chunk.nbits)
    seq_tile_size = property(lambda self: self.chunk.seq_tile)
    head_dim = property(lambda self: self.chunk.head_dim)

    @property
    def original_shape(self) -> tuple:
        c = self.chunk
        return (c.batch, c.heads, c.seq_tile, c.head_dim)

    @property
    def n_elements(self) -> int:
        c = self.chunk
        return c.batch * c.heads * c.seq_tile * c.head_dim

    @property
    def n_escapes(self) -> int:
        off = self.chunk.seg_offsets
        return int(off[self.j + 1]) - int(off[self.j])

    def view(self) -> TiledCompressedTensor:
        return self.chunk.segment(self.j)

    # tensor fields, for code written against TiledCompressedTensor
    sign_mass_data = property(lambda self: self.view().sign_mass_data)
    exp_data = property(lambda self: self.view().exp_data)
    invalid_exp = property(lambda self: self.view().invalid_exp)
    tile_invalid_base = property(lambda self: self.view().tile_invalid_base)

    def get_memory(self) -> dict:
        """compress_tiled_kv.py:269-282, without touching a tensor."""
        c = self.chunk
        n = self.n_elements
        compressed = n + n * c.nbits // 8 + self.n_escapes + 4 * c.batch * c.heads
        return {'compressed_memory': compressed, 'original_memory': 2 * n,
                'ratio': 0.0 if n == 0 else compressed / (2 * n)}

    def export_state(self) -> dict:
        return self.view().export_state()

    def export_decode_view(self) -> dict:
        return self.view().export_decode_view()

    def materialize(self) -> torch.Tensor:
        return self.view().materialize()


@dataclass
class PackedChunk:
    """``n_blocks`` consecutive segments produced by one pack launch with one window.
    Plane tensors are segment-major; ``segment(j)`` gives views shaped like the reference's
    per-block ``TiledCompressedTensor``."""

    sign_mant: torch.Tensor      # uint8 [n_blocks, B*H*tile_elems]
    codes: torch.Tensor          # uint8 [n_blocks, B*H*tile_elems*nbits/8]
    escapes: torch.Tensor        # uint8 [n_escapes]
    tile_base: torch.Tensor      # int32 [n_blocks, B*H]
    seg_offsets: list            # host ints, n_blocks + 1
    seg_offsets_dev: torch.Tensor  # the same, int64 on the device
    left: int
    right: int
    nbits: int
    batch: int
    heads: int
    seq_tile: int
    head_dim: int
    _segments: dict = field(default_factory=dict, repr=False)

    @property
    def n_blocks(self) -> int:
        return int(self.sign_mant.shape[0])

    @property
    def n_escapes(self) -> int:
        return int(self.seg_offsets[-1])

    def segment(self, j: int) -> TiledCompressedTensor:
        seg = self._segments.get(j)
        if seg is None:
            lo, hi = int(self.seg_offsets[j]), int(self.seg_offsets[j + 1])
            seg = TiledCompressedTensor(
                sign_mass_data=self.sign_mant[j], exp_data=self.codes[j], invalid_exp=self.escapes[lo:hi],
                tile_invalid_base=self.tile_base[j], left=self.left, right=self.right, nbits=self.nbits,
                original_shape=(self.batch, self.heads, self.seq_tile, self.head_dim),
                seq_tile_size=self.seq_tile, head_dim=self.head_dim, tile_head_dim=self.head_dim,
                tile_num_lanes=self.head_dim // 8, num_sequence_tiles=1, num_kv_heads=self.heads,
                device=self.sign_mant.device)
            self._segments[j] = seg
        return seg

    def segments(self) -> list:
        """Cheap handles, one per block (``SegmentRef``)."""
        return [SegmentRef(self, j) for j in range(self.n_blocks)]


# --------------------------------------------------------------------------------------
# kernels
# --------------------------------------------------------------------------------------

def _check_src(x: torch.Tensor) -> torch.Tensor:
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    if x.dim() != 4:
        raise ValueError(f'Expected 4D [batch, kv_heads, seq, head_dim] tensor, got {tuple(x.shape)}')
    if x.shape[-1] % 8 != 0:
        raise ValueError(f'Tiled compressed path requires head_dim % 8 == 0, got {x.shape[-1]}')
    sb, sh, ss, sd = x.stride()
    if x.numel() and (sd != 1 or (sb | sh | ss) % 8 != 0 or x.data_ptr() % 16 != 0):
        x = x.contiguous()
    return x


class _PendingPack:
    """A pack launch whose escape totals have not been read yet (``pack_blocks_launch``)."""

    def __init__(self, **kw):
        self.__dict__.update(kw)


def _default_escape_capacity(n: int) -> int:
    return min(max(4096, n // 8), max(n, 1))


def pack_blocks_launch(x: torch.Tensor, right: int, nbits: int, seq_tile: int = 128, need_hist: bool = False,
                       hist_out: Optional[torch.Tensor] = None, escape_capacity: Optional[int] = None,
                       meta_out: Optional[torch.Tensor] = None, launch: bool = True) -> _PendingPack:
    """Start packing ``x`` (see ``pack_blocks``) and return without reading anything back.
    ``meta_out``: zeroed int64[n_blocks + 2] device buffer for the segment offsets and the status
    word (e.g. a slice of a buffer that several launches share, so that one ``read_back`` serves
    them all); the caller passes its host copy to ``pack_blocks_finish``."""
    if nbits not in _SUPPORTED_TILE_NBITS:
        raise ValueError(f'Tiled compressed path supports nbits in {_SUPPORTED_TILE_NBITS}, got {nbits}')
    x = _check_src(x)
    B, H, S, D = x.shape
    if seq_tile <= 0:
        raise ValueError('seq_tile_size must be positive')
    if S % seq_tile != 0:
        raise ValueError(f'sequence length {S} is not a multiple of seq_tile_size {seq_tile}')
    n_blocks = S // seq_tile
    dev = x.device
    tile_elems = seq_tile * D
    n = B * H * n_blocks * tile_elems
    p = _PendingPack(x=x, right=int(right), nbits=int(nbits), seq_tile=seq_tile, B=B, H=H, D=D, n_blocks=n_blocks,
                     dev=dev, n=n)
    p.sign_mant = torch.empty((n_blocks, B * H * tile_elems), dtype=torch.uint8, device=dev)
    p.codes = torch.empty((n_blocks, B * H * tile_elems * nbits // 8), dtype=torch.uint8, device=dev)
    p.tile_base = torch.empty((n_blocks, B * H), dtype=torch.int32, device=dev)
    # [segment offsets (n_blocks+1) | status word] in one int64 buffer -> one read
    p.meta = meta_out if meta_out is not None else torch.zeros(n_blocks + 2, dtype=torch.int64, device=dev)
    if p.meta.numel() != n_blocks + 2 or p.meta.dtype != torch.int64 or not p.meta.is_contiguous():
        raise ValueError('meta_out must be a contiguous int64 tensor of n_blocks + 2 entries')
    p.hist = None
    if need_hist:
        p.hist = hist_out if hist_out is not None else torch.zeros(256, dtype=torch.int32, device=dev)
    p.cap = min(int(escape_capacity), max(n, 1)) if escape_capacity is not None else _default_escape_capacity(n)
    if launch:
        p.escapes = _pack_launch(p, p.cap, p.hist)
    return p


def _pack_launch(p: _PendingPack, capacity: int, hist_t) -> torch.Tensor:
    sc = _scratch_for(p.dev)
    n_tiles = p.B * p.H * p.n_blocks
    ws = sc.workspace_for(n_tiles, p.seq_tile * p.D)
    esc = torch.empty(capacity, dtype=torch.uint8, device=p.dev)
    sb, sh, ss, _ = p.x.stride()
    with torch.cuda.device(p.dev):
        rc = _lib.lib().adacode_pack_tiles(
            p.x.data_ptr(), sb, sh, ss, p.B, p.H, p.n_blocks, p.seq_tile, p.D, p.right, p.nbits,
            p.sign_mant.data_ptr(), p.codes.data_ptr(), esc.data_ptr(), capacity, p.tile_base.data_ptr(),
            p.meta.data_ptr(), 0 if hist_t is None else hist_t.data_ptr(), ws.data_ptr(), ws.numel(),
            p.meta.data_ptr() + 8 * (p.n_blocks + 1), _stream_ptr(p.dev))
    _lib.check(rc, 'adacode_pack_tiles')
    return esc


def _pack_launch_jobs(ps: Sequence[_PendingPack]) -> None:
    """One ``adacode_pack_jobs`` launch for pending packs of one shape and code length (the keys and
    the values of a span); every pack gets its own escape buffer, the status word is the first one's."""
    first = ps[0]
    dev = first.dev
    sc = _scratch_for(dev)
    n_tiles = sum(p.B * p.H * p.n_blocks for p in ps)
    ws = sc.workspace_for(n_tiles, first.seq_tile * first.D)
    jobs = (_lib.PackJob * len(ps))()
    for jb, p in zip(jobs, ps):
        p.escapes = torch.empty(p.cap, dtype=torch.uint8, device=dev)
        sb, sh, ss, _ = p.x.stride()
        jb.src_bf16, jb.stride_b, jb.stride_h, jb.stride_s = p.x.data_ptr(), sb, sh, ss
        jb.n_blocks, jb.right = p.n_blocks, p.right
        jb.sign_mant, jb.codes, jb.escapes = p.sign_mant.data_ptr(), p.codes.data_ptr(), p.escapes.data_ptr()
        jb.escapes_capacity = p.cap
        jb.tile_base, jb.seg_escape_offsets = p.tile_base.data_ptr(), p.meta.data_ptr()
        jb.hist256 = 0 if p.hist is None else p.hist.data_ptr()
    with torch.cuda.device(dev):
        rc = _lib.lib().adacode_pack_jobs(
            ctypes.addressof(jobs), len(ps), first.B, first.H, first.seq_tile, first.D, first.nbits,
            ws.data_ptr(), ws.numel(), first.meta.data_ptr() + 8 * (first.n_blocks + 1), _stream_ptr(dev))
    _lib.check(rc, 'adacode_pack_jobs')


def pack_blocks_finish(p: _PendingPack, host_meta):
    """Finish a launch given the host copy of its ``meta`` (int64[n_blocks + 2]): re-run with the
    exact capacity if the escape buffer was too small, trim it, build the ``PackedChunk``."""
    n_blocks = p.n_blocks
    offsets = [int(v) for v in host_meta[: n_blocks + 1]]
    total = offsets[-1]
    status = int(host_meta[n_blocks + 1]) & 0xFFFFFFFF
    escapes = p.escapes
    # the kernels flag an overflow exactly when a stream does not fit its buffer; packs that shared
    # a launch share the status word, so each one decides by its own total
    status_other = status & ~_lib.STATUS_ESCAPE_OVERFLOW
    if total > p.cap:
        p.meta.zero_()
        escapes = _pack_launch(p, total, None)   # histogram already complete from the first pass
        host = read_back(p.meta)
        if int(host[n_blocks + 1]) & 0xFFFFFFFF:
            raise _lib.AdacodeError('adacode_pack_tiles: escape overflow after re-run with exact capacity')
    elif status_other:
        raise _lib.AdacodeError(f'adacode_pack_tiles: device status {status:#x} ({describe_status(status)})')
    if escapes.numel() > 2 * total + 65536:
        escapes = escapes[:total].clone()
    else:
        escapes = escapes[:total]
    chunk = PackedChunk(p.sign_mant, p.codes, escapes, p.tile_base, offsets, p.meta[: n_blocks + 1],
                        p.right - 2 ** p.nbits + 1, p.right, p.nbits, p.B, p.H, p.seq_tile, p.D)
    return chunk, p.hist


def pack_blocks(x: torch.Tensor, right: int, nbits: int, seq_tile: int = 128, need_hist: bool = False,
                hist_out: Optional[torch.Tensor] = None, escape_capacity: Optional[int] = None):
    """Pack ``x`` [B, H, n_blocks*seq_tile, D] (bf16, any B/H/S strides) into ``n_blocks`` segments
    with the window ``(right - 2**nbits + 1, right]`` in one launch.

    Returns ``(PackedChunk, hist)``; ``hist`` is an int32[256] device tensor of all exponents when
    ``need_hist`` (``hist_out`` is added to instead when given).  One small device-to-host read
    (segment escape totals and the status word) ends the call.
    """
    p = pack_blocks_launch(x, right, nbits, seq_tile, need_hist, hist_out, escape_capacity)
    return pack_blocks_finish(p, read_back(p.meta))


def pack_pair(k: torch.Tensor, v: torch.Tensor, k_params, v_params, seq_tile: int = 128, need_hist: bool = False,
              capacities=(None, None)):
    """Pack the keys and the values of one span with one round trip to the host: both launches
    write their segment offsets, status words and (with ``need_hist``) exponent histograms into
    one device buffer that a single ``read_back`` fetches.  Returns
    ``(k_chunk, v_chunk, k_hist, v_hist, k_hist_host, v_hist_host)``; the ``*_host`` entries are
    numpy int32[256] copies of the histograms (None without ``need_hist``)."""
    dev = k.device
    nk = k.shape[-2] // seq_tile + 2
    nv = v.shape[-2] // seq_tile + 2
    words = nk + nv + (256 if need_hist else 0)          # int64 words; two int32[256] histograms = 256 words
    mail = torch.zeros(words, dtype=torch.int64, device=dev)
    k_hist = v_hist = None
    if need_hist:
        h = mail[nk + nv:].view(torch.int32)
        k_hist, v_hist = h[:256], h[256:]
    # keys and values of one shape and code length go through ONE launch (their windows may differ)
    together = (tuple(k.shape) == tuple(v.shape) and int(k_params[1]) == int(v_params[1]) and k.numel() > 0
                and k.shape[-1] % 8 == 0 and 2 * k.numel() < 2 ** 31)
    pk = pack_blocks_launch(k, k_params[0], k_params[1], seq_tile, need_hist, k_hist, capacities[0], mail[:nk],
                            launch=not together)
    pv = pack_blocks_launch(v, v_params[0], v_params[1], seq_tile, need_hist, v_hist, capacities[1],
                            mail[nk:nk + nv], launch=not together)
    if together:
        _pack_launch_jobs([pk, pv])
    host = read_back(mail)
    if together:
        # one status word (the keys') serves both packs
        host[nk + nv - 1] = int(host[nk + nv - 1]) | int(host[nk - 1])
    k_chunk, _ = pack_blocks_finish(pk, host[:nk])
    v_chunk, _ = pack_blocks_finish(pv, host[nk:nk + nv])
    kh = vh = None
    if need_hist:
        hh = host[nk + nv:].view('int32')
        kh, vh = hh[:256].copy(), hh[256:].copy()
    return k_chunk, v_chunk, k_hist, v_hist, kh, vh


def unpack_chunk(chunk: PackedChunk, dst: torch.Tensor, seq_offset: int = 0) -> None:
    """Unpack every segment of ``chunk`` into ``dst[:, :, seq_offset : seq_offset + n_blocks*seq_tile]``."""
    B, H, T, D = chunk.batch, chunk.heads, chunk.seq_tile, chunk.head_dim
    _check_dst(dst, B, H, D, seq_offset + chunk.n_blocks * T)
    dev = dst.device
    sc = _scratch_for(dev)
    view = dst[:, :, seq_offset:]
    db, dh, ds, _ = dst.stride()
    seg_off = chunk.seg_offsets_dev
    with torch.cuda.device(dev):
        rc = _lib.lib().adacode_unpack_tiles(
            chunk.sign_mant.data_ptr(), chunk.codes.data_ptr(), chunk.escapes.data_ptr(), chunk.escapes.numel(),
            chunk.tile_base.data_ptr(), seg_off.data_ptr(), B, H, chunk.n_blocks, T, D,
            chunk.left, chunk.nbits, view.data_ptr(), db, dh, ds, sc.status.data_ptr(), _stream_ptr(dev))
    _lib.check(rc, 'adacode_unpack_tiles')


def _check_dst(dst: torch.Tensor, B: int, H: int, D: int, min_seq: int) -> None:
    if dst.dtype != torch.bfloat16 or dst.dim() != 4:
        raise ValueError(f'dst must be a 4D bf16 tensor, got {dst.dtype} {tuple(dst.shape)}')
    if dst.shape[0] != B or dst.shape[1] != H or dst.shape[3] != D or dst.shape[2] < min_seq:
        raise ValueError(f'dst shape {tuple(dst.shape)} cannot hold [{B}, {H}, {min_seq}, {D}]')
    if dst.stride(3) != 1:
        raise ValueError('dst must have unit stride along head_dim')


_SEGMENT_DTYPE = None


def _segment_dtype():
    """numpy mirror of ``struct adacode_segment`` (56 bytes)."""
    global _SEGMENT_DTYPE
    if _SEGMENT_DTYPE is None:
        import numpy as np
        _SEGMENT_DTYPE = np.dtype([('sign_mant', '<u8'), ('codes', '<u8'), ('escapes', '<u8'), ('tile_base', '<u8'),
                                   ('escapes_len', '<i8'), ('dst_seq_offset', '<i8'), ('left', '<i4'),
                                   ('nbits', '<i4')])
        assert _SEGMENT_DTYPE.itemsize == ctypes.sizeof(_lib.Segment)
    return _SEGMENT_DTYPE


def _check_segment_buffers(seg) -> None:
    """A segment record carries raw pointers: refuse on the host what would fault on the device."""
    B, H, T, D = (int(v) for v in seg.original_shape)
    n = B * H * T * D
    nbits = int(seg.nbits)
    if nbits not in _SUPPORTED_TILE_NBITS:
        raise ValueError(f'Tiled compressed path supports nbits in {_SUPPORTED_TILE_NBITS}, got {nbits}')
    if seg.sign_mass_data.dtype != torch.uint8 or seg.sign_mass_data.numel() < n:
        raise ValueError(f'segment sign_mass_data must hold {n} uint8 values, got {seg.sign_mass_data.numel()}')
    if seg.exp_data.dtype != torch.uint8 or seg.exp_data.numel() < n * nbits // 8:
        raise ValueError(f'segment exp_data must hold {n * nbits // 8} uint8 values, got {seg.exp_data.numel()}')
    base = seg.tile_invalid_base
    if base.dtype != torch.int32 or base.numel() < B * H or not base.is_contiguous():
        raise ValueError(f'segment tile_invalid_base must be {B * H} contiguous int32 values, got '
                         f'{base.numel()} of {base.dtype}')
    if n and (seg.sign_mass_data.data_ptr() % 16 or seg.exp_data.data_ptr() % 16):
        raise ValueError('segment planes must start on 16-byte boundaries')
    if seg.invalid_exp.numel() and seg.invalid_exp.dtype != torch.uint8:
        raise ValueError('segment invalid_exp must be uint8')


def build_segment_table(segments: Sequence, seq_offsets: Optional[Sequence[int]] = None,
                        device=None) -> torch.Tensor:
    """Device array of ``adacode_segment`` records (as uint8) for ``unpack_segments``.
    ``seq_offsets[i]`` is segment i's first token in the destination; the default stacks the
    segments one after the other.  Runs of ``SegmentRef`` from one chunk are filled with array
    arithmetic on the chunk's base pointers, so a table over hundreds of blocks costs a handful
    of numpy operations."""
    import numpy as np
    n = len(segments)
    table = np.zeros(max(n, 1), dtype=_segment_dtype())
    i = 0
    run_tokens = 0
    while i < n:
        seg = segments[i]
        if isinstance(seg, SegmentRef):
            c = seg.chunk
            k = i + 1
            while k < n and isinstance(segments[k], SegmentRef) and segments[k].chunk is c \
                    and segments[k].j == segments[k - 1].j + 1:
                k += 1
            js = np.arange(seg.j, seg.j + (k - i), dtype=np.int64)
            offs = np.asarray(c.seg_offsets, dtype=np.int64)
            bh = c.batch * c.heads
            tile = c.seq_tile * c.head_dim
            rows = table[i:k]
            rows['sign_mant'] = c.sign_mant.data_ptr() + js * (bh * tile)
            rows['codes'] = c.codes.data_ptr() + js * (bh * tile * c.nbits // 8)
            esc_base = c.escapes.data_ptr() if c.escapes.numel() else 0
            lens = offs[js + 1] - offs[js]
            rows['escapes'] = np.where(lens > 0, esc_base + offs[js], 0)
            rows['tile_base'] = c.tile_base.data_ptr() + js * (4 * bh)
            rows['escapes_len'] = lens
            rows['left'] = c.left
            rows['nbits'] = c.nbits
            tokens = np.full(k - i, c.seq_tile, dtype=np.int64)
        else:
            k = i + 1
            rows = table[i:k]
            _check_segment_buffers(seg)
            rows['sign_mant'] = seg.sign_mass_data.data_ptr()
            rows['codes'] = seg.exp_data.data_ptr()
            rows['escapes'] = seg.invalid_exp.data_ptr() if seg.invalid_exp.numel() else 0
            rows['tile_base'] = seg.tile_invalid_base.data_ptr()
            rows['escapes_len'] = seg.invalid_exp.numel()
            rows['left'] = int(seg.left)
            rows['nbits'] = int(seg.nbits)
            tokens = np.asarray([int(seg.original_shape[-2])], dtype=np.int64)
        if seq_offsets is None:
            starts = run_tokens + np.concatenate(([0], np.cumsum(tokens)[:-1]))
            run_tokens += int(tokens.sum())
        else:
            starts = np.asarray([int(v) for v in seq_offsets[i:k]], dtype=np.int64)
            run_tokens = int(starts[-1] + tokens[-1])
        rows['dst_seq_offset'] = starts
        i = k
    host = torch.from_numpy(table[:n].view(np.uint8).reshape(-1).copy()) if n else torch.empty(0, dtype=torch.uint8)
    if device is None:
        s0 = segments[0]
        device = s0.chunk.sign_mant.device if isinstance(s0, SegmentRef) else s0.sign_mass_data.device
    return host.to(device, non_blocking=False)


def unpack_segments(segments: Sequence[TiledCompressedTensor], dst: torch.Tensor,
                    seq_offsets: Optional[Sequence[int]] = None, table: Optional[torch.Tensor] = None) -> None:
    """Unpack a list of segments (any mix of windows and code lengths) into ``dst`` [B, H, S, D]
    with one launch.  Replaces the reference's per-segment decode + ``torch.cat``
    (float_cache_utils.py:1257-1264)."""
    if not segments:
        return
    first = segments[0]
    B, H, T, D = first.original_shape
    for seg in segments:
        if tuple(seg.original_shape) != (B, H, T, D):
            raise ValueError('all segments of one call must share [batch, kv_heads, seq_tile, head_dim]')
    _check_dst(dst, B, H, D, 0)
    dev = dst.device
    sc = _scratch_for(dev)
    if table is None:
        table = build_segment_table(segments, seq_offsets, dev)
    db, dh, ds, _ = dst.stride()
    with torch.cuda.device(dev):
        rc = _lib.lib().adacode_unpack_segments(table.data_ptr(), len(segments), B, H, T, D, dst.data_ptr(),
                                                db, dh, ds, sc.status.data_ptr(), _stream_ptr(dev))
    _lib.check(rc, 'adacode_unpack_segments')


def unpack_segments_multi(jobs: Sequence[tuple]) -> None:
    """Unpack several segment lists, each into its own destination, with ONE launch when they
    share [batch, kv_heads, seq_tile, head_dim] (the keys and the values of a layer).
    ``jobs``: ``(segments, dst, table_or_None)`` tuples; anything that does not fit one launch
    falls back to one ``unpack_segments`` call per entry."""
    jobs = [j for j in jobs if j[0]]
    if not jobs:
        return
    shape0 = tuple(jobs[0][0][0].original_shape)
    same = all(tuple(seg.original_shape) == shape0 for segs, _, _ in jobs for seg in (segs[0], segs[-1]))
    if len(jobs) == 1 or not same or len(jobs) > int(_lib.lib().adacode_max_jobs()):
        for segs, dst, table in jobs:
            unpack_segments(segs, dst, table=table)
        return
    B, H, T, D = shape0
    dev = jobs[0][1].device
    sc = _scratch_for(dev)
    arr = (_lib.UnpackJob * len(jobs))()
    keep = []
    for rec, (segs, dst, table) in zip(arr, jobs):
        for seg in segs:
            if tuple(seg.original_shape) != shape0:
                raise ValueError('all segments of one call must share [batch, kv_heads, seq_tile, head_dim]')
        _check_dst(dst, B, H, D, 0)
        if table is None:
            table = build_segment_table(segs, None, dev)
        keep.append(table)
        db, dh, ds, _ = dst.stride()
        rec.segments_dev, rec.n_segments = table.data_ptr(), len(segs)
        rec.dst_bf16, rec.dstride_b, rec.dstride_h, rec.dstride_s = dst.data_ptr(), db, dh, ds
    with torch.cuda.device(dev):
        rc = _lib.lib().adacode_unpack_jobs(ctypes.addressof(arr), len(jobs), B, H, T, D, sc.status.data_ptr(),
                                            _stream_ptr(dev))
    _lib.check(rc, 'adacode_unpack_jobs')


def exponent_hist(x: torch.Tensor, hist_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """int32[256] device histogram of the exponent field of ``x`` [B, H, S, D]
    (float_cache_utils.py:883-891)."""
    x = _check_src(x)
    dev = x.device
    _scratch_for(dev)
    hist = hist_out if hist_out is not None else torch.zeros(256, dtype=torch.int32, device=dev)
    B, H, S, D = x.shape
    sb, sh, ss, _ = x.stride()
    with torch.cuda.device(dev):
        rc = _lib.lib().adacode_hist_bf16(x.data_ptr(), sb, sh, ss, B, H, S, D, hist.data_ptr(), _stream_ptr(dev))
    _lib.check(rc, 'adacode_hist_bf16')
    return hist


def choose_params_device(hists: torch.Tensor) -> torch.Tensor:
    """(right, nbits) pairs, int32 [n, 2] on the device, for int32 histograms [n, 256];
    nbits == 0 marks a histogram for which no code length beats 8 bits."""
    if hists.dtype != torch.int32 or hists.shape[-1] != 256:
        raise ValueError('expected int32 histograms with 256 bins')
    h = hists.reshape(-1, 256).contiguous()
    dev = h.device
    _scratch_for(dev)
    out = torch.empty((h.shape[0], 2), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().adacode_choose_params(h.data_ptr(), h.shape[0], out.data_ptr(), _stream_ptr(dev))
    _lib.check(rc, 'adacode_choose_params')
    return out


def analysis_best_bits(data_freq, store_index: bool = False):
    """(right, nbits) for one 256-bin histogram given as a tensor, array or list on the host
    (float_cache_utils.py:373-398).  Raises IndexError where the reference does."""
    if store_index:
        raise NotImplementedError('store_index=True is not used by the float11 cache path')
    values = data_freq.tolist() if hasattr(data_freq, 'tolist') else list(data_freq)
    if len(values) != 256:
        raise ValueError(f'expected 256 bins, got {len(values)}')
    arr = (ctypes.c_int64 * 256)(*[int(v) for v in values])
    r, n = ctypes.c_int(0), ctypes.c_int(0)
    rc = _lib.lib().adacode_choose_params_host(arr, ctypes.byref(r), ctypes.byref(n))
    if rc == _lib.ERR_NO_CANDIDATE:
        raise IndexError('list index out of range')
    _lib.check(rc, 'adacode_choose_params_host')
    return int(r.value), int(n.value)


# --------------------------------------------------------------------------------------
# reference-shaped entry points
# --------------------------------------------------------------------------------------

def compress_tiled_tensor(original_data_bfloat16: torch.Tensor, right: int, nbits: int = _DEFAULT_TILE_NBITS,
                          seq_tile_size: int = 128, tile_head_dim: Optional[int] = None,
                          need_adjust: bool = False):
    """Pack exactly one block; same arguments, checks and return value as the reference
    (compress_tiled_kv.py:591-630)."""
    if nbits not in _SUPPORTED_TILE_NBITS:
        raise ValueError(f'Tiled compressed path supports nbits in {_SUPPORTED_TILE_NBITS}, got {nbits}')
    if original_data_bfloat16.dtype != torch.bfloat16:
        original_data_bfloat16 = original_data_bfloat16.to(torch.bfloat16)
    if original_data_bfloat16.dim() != 4:
        raise ValueError(
            f'Expected 4D [batch, kv_heads, seq, head_dim] tensor, got {tuple(original_data_bfloat16.shape)}')
    _, _, seq_len, head_dim = original_data_bfloat16.shape
    if seq_tile_size <= 0:
        raise ValueError('seq_tile_size must be positive')
    if tile_head_dim is None:
        tile_head_dim = head_dim
    if tile_head_dim != head_dim:
        raise ValueError(
            f'Tiled compressed path currently requires tile_head_dim == head_dim, got {tile_head_dim} vs {head_dim}')
    if head_dim % 8 != 0:
        raise ValueError(f'Tiled compressed path requires head_dim % 8 == 0, got {head_dim}')
    if seq_tile_size != seq_len:
        raise ValueError(
            'Tiled compressed path currently requires seq_tile_size == seq_len per compressed block, '
            f'got seq_tile_size={seq_tile_size}, seq_len={seq_len}')
    chunk, hist = pack_blocks(original_data_bfloat16, right, nbits, seq_tile_size, need_hist=need_adjust)
    return chunk.segment(0), hist


def tensor_from_state(state: dict) -> TiledCompressedTensor:
    dev = state['device']
    return TiledCompressedTensor(
        sign_mass_data=state['sign_mass_data'], exp_data=state['exp_data'],
        invalid_exp=state.get('invalid_exp', torch.empty((0,), dtype=torch.uint8, device=dev)),
        tile_invalid_base=state.get('tile_invalid_base', torch.empty((0,), dtype=torch.int32, device=dev)),
        left=state['left'], right=state['right'], nbits=state['nbits'],
        original_shape=tuple(state['original_shape']), seq_tile_size=state['seq_tile_size'],
        head_dim=state['head_dim'], tile_head_dim=state['tile_head_dim'],
        tile_num_lanes=state['tile_num_lanes'],
        num_sequence_tiles=int(state.get('num_sequence_tiles', 1)), num_kv_heads=state['num_kv_heads'],
        device=dev)


def materialize_tiled_state(state: dict) -> torch.Tensor:
    """Dense bf16 tensor of one exported segment state (compress_tiled_kv.py:754-791)."""
    if state.get('layout') == 'tiled_open_rows':
        raise NotImplementedError('open-row tiles are not produced by the segmented_tiled cache path')
    return tensor_from_state(state).materialize()

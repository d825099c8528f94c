"""ctypes binding of ``libadacode_sm100.so`` (the C ABI in ``include/adacode.h``).

There is no fallback: if the library has not been built, or a call fails, an exception is
raised.  The library is loaded on first use so that the host-side classes can be imported
(and their pure-Python logic tested) on a machine without the built artefact.
"""
from __future__ import annotations

import ctypes
import os

from .build import LIB_PATH

OK = 0
ERR_INVALID_ARG = -1
ERR_CUDA = -2
ERR_WORKSPACE = -3
ERR_NO_CANDIDATE = -4
ERR_TOO_LARGE = -5
STATIC_SCRATCH_BYTES = 4 * 1024 * 1024 + 512 * 1024
STATUS_ESCAPE_OVERFLOW = 1
STATUS_ESCAPE_UNDERRUN = 2
STATUS_TIMEOUT = 4
STATUS_MISALIGNED = 8

# every symbol include/adacode.h declares
EXPORTED_SYMBOLS = (
    'adacode_version', 'adacode_strerror', 'adacode_last_cuda_error', 'adacode_pack_workspace_bytes',
    'adacode_pack_tiles', 'adacode_unpack_tiles', 'adacode_unpack_segments', 'adacode_hist_bf16',
    'adacode_choose_params', 'adacode_choose_params_host', 'adacode_calibrate_host', 'adacode_pack_tiles_static',
    'adacode_decode_attn_workspace_bytes', 'adacode_decode_attn', 'adacode_copy_to_host',
    'adacode_pack_jobs', 'adacode_unpack_jobs', 'adacode_max_jobs', 'adacode_debug_set_wait_limit',
    'adacode_flat_block_elems', 'adacode_unpack_flat',
)


class Segment(ctypes.Structure):
    """Mirror of ``struct adacode_segment``."""
    _fields_ = [
        ('sign_mant', ctypes.c_void_p), ('codes', ctypes.c_void_p), ('escapes', ctypes.c_void_p),
        ('tile_base', ctypes.c_void_p), ('escapes_len', ctypes.c_int64), ('dst_seq_offset', ctypes.c_int64),
        ('left', ctypes.c_int32), ('nbits', ctypes.c_int32),
    ]


class PackJob(ctypes.Structure):
    """Mirror of ``struct adacode_pack_job``."""
    _fields_ = [
        ('src_bf16', ctypes.c_void_p), ('stride_b', ctypes.c_int64), ('stride_h', ctypes.c_int64),
        ('stride_s', ctypes.c_int64), ('n_blocks', ctypes.c_int32), ('right', ctypes.c_int32),
        ('sign_mant', ctypes.c_void_p), ('codes', ctypes.c_void_p), ('escapes', ctypes.c_void_p),
        ('escapes_capacity', ctypes.c_int64), ('tile_base', ctypes.c_void_p),
        ('seg_escape_offsets', ctypes.c_void_p), ('hist256', ctypes.c_void_p),
    ]


class UnpackJob(ctypes.Structure):
    """Mirror of ``struct adacode_unpack_job``."""
    _fields_ = [
        ('segments_dev', ctypes.c_void_p), ('n_segments', ctypes.c_int32), ('reserved', ctypes.c_int32),
        ('dst_bf16', ctypes.c_void_p), ('dstride_b', ctypes.c_int64), ('dstride_h', ctypes.c_int64),
        ('dstride_s', ctypes.c_int64),
    ]


class AdacodeError(RuntimeError):
    pass


_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it was never built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise AdacodeError(
            f'{LIB_PATH} is missing: build it with `python -m adacode_b200.build` '
            '(nvcc, sm_100a). This package has no CPU or Triton fallback.')
    L = ctypes.CDLL(LIB_PATH)
    vp, i64, i32, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
    L.adacode_version.restype = i32
    L.adacode_strerror.restype = ctypes.c_char_p
    L.adacode_strerror.argtypes = [i32]
    L.adacode_last_cuda_error.restype = ctypes.c_char_p
    L.adacode_pack_workspace_bytes.restype = sz
    L.adacode_pack_workspace_bytes.argtypes = [i64, i64]
    L.adacode_pack_tiles.restype = i32
    L.adacode_pack_tiles.argtypes = [vp, i64, i64, i64, i32, i32, i32, i32, i32, i32, i32,
                                     vp, vp, vp, i64, vp, vp, vp, vp, sz, vp, vp]
    L.adacode_pack_tiles_static.restype = i32
    L.adacode_pack_tiles_static.argtypes = [vp, i64, i64, i64, i32, i32, i32, i32, i32, i32, i32,
                                            vp, vp, vp, i64, vp, vp, vp, vp, vp]
    L.adacode_unpack_tiles.restype = i32
    L.adacode_unpack_tiles.argtypes = [vp, vp, vp, i64, vp, vp, i32, i32, i32, i32, i32, i32, i32,
                                       vp, i64, i64, i64, vp, vp]
    L.adacode_unpack_segments.restype = i32
    L.adacode_unpack_segments.argtypes = [vp, i32, i32, i32, i32, i32, vp, i64, i64, i64, vp, vp]
    L.adacode_hist_bf16.restype = i32
    L.adacode_hist_bf16.argtypes = [vp, i64, i64, i64, i32, i32, i32, i32, vp, vp]
    L.adacode_choose_params.restype = i32
    L.adacode_choose_params.argtypes = [vp, i32, vp, vp]
    L.adacode_choose_params_host.restype = i32
    L.adacode_choose_params_host.argtypes = [vp, ctypes.POINTER(i32), ctypes.POINTER(i32)]
    L.adacode_calibrate_host.restype = i32
    L.adacode_calibrate_host.argtypes = [vp, ctypes.POINTER(i32), ctypes.POINTER(i32)]
    L.adacode_decode_attn_workspace_bytes.restype = sz
    L.adacode_decode_attn_workspace_bytes.argtypes = [i32, i32, i32, i32]
    L.adacode_decode_attn.restype = i32
    L.adacode_decode_attn.argtypes = [vp, i64, i64, vp, vp, i32, vp, vp, i32, i64, i64, i64,
                                      i32, i32, i32, i32, i32, ctypes.c_float, vp, vp, sz, i32, vp, vp]
    L.adacode_copy_to_host.restype = i32
    L.adacode_copy_to_host.argtypes = [vp, vp, sz, vp]
    L.adacode_max_jobs.restype = i32
    L.adacode_flat_block_elems.restype = i32
    L.adacode_flat_block_elems.argtypes = [i32]
    L.adacode_unpack_flat.restype = i32
    L.adacode_unpack_flat.argtypes = [vp, vp, vp, i64, vp, i64, i32, i32, vp, vp, vp]
    L.adacode_debug_set_wait_limit.restype = i32
    L.adacode_debug_set_wait_limit.argtypes = [ctypes.c_uint, i32]
    L.adacode_pack_jobs.restype = i32
    L.adacode_pack_jobs.argtypes = [vp, i32, i32, i32, i32, i32, i32, vp, sz, vp, vp]
    L.adacode_unpack_jobs.restype = i32
    L.adacode_unpack_jobs.argtypes = [vp, i32, i32, i32, i32, i32, vp, vp]
    _lib = L
    return L


def check(rc: int, what: str) -> None:
    """Raise for a non-zero return code of the library."""
    if rc == OK:
        return
    L = lib()
    msg = L.adacode_strerror(rc).decode()
    if rc == ERR_CUDA:
        msg += ': ' + L.adacode_last_cuda_error().decode()
    if rc == ERR_INVALID_ARG:
        raise ValueError(f'{what}: {msg}')
    raise AdacodeError(f'{what}: {msg}')

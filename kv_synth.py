"""Seeded synthetic KV tensors whose BYTES are the same on every device.

The benchmark compares a GPU arm and a CPU arm on the same workload, and multi-GPU runs compare
shards with an unsharded oracle run, so the generator must give identical bf16 bit patterns
whether it runs as CUDA kernels or on host cores, for the whole tensor or for any slab of it.
``torch.randn`` cannot do that (different generators per device), and transcendental functions
round differently on CPU and GPU.  So every element is a pure function of its coordinates:

    u      = mix64(seed, layer, which, b, h, s, d)          integer hash (wrapping int64 arithmetic)
    z      = QUANTILE[u >> 48]                               65 536-entry table of N(0, 1) quantiles (fp32)
    x      = bf16(z * sigma[h, d] + offset[h, d])            one fp32 multiply, one fp32 add, one rounding

with the small per-channel tables ``sigma`` / ``offset`` drawn once from a CPU generator.  The value
distributions are those the benchmark configurations name: sigma_c ~ LogNormal(mu, s), 2 % outlier
channels scaled x30, a per-channel offset ~ N(0, 2) on keys, an optional sigma x2 for half the
heads from some token on, and optional injected escapes (a Bernoulli subset of exponent fields
replaced by values outside a window, another set to zero).  No dataset item is reproduced.
"""
from __future__ import annotations

import math

import torch

_MASK63 = (1 << 63) - 1


def _c(v: int) -> int:
    """A 64-bit constant as the signed value torch.int64 wants."""
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


_M1, _M2, _GOLD = _c(0xBF58476D1CE4E5B9), _c(0x94D049BB133111EB), _c(0x9E3779B97F4A7C15)


def _mix(x: torch.Tensor) -> torch.Tensor:
    """splitmix64 finaliser on an int64 tensor (logical shifts emulated by masking the sign extension)."""
    x = (x ^ ((x >> 30) & ((1 << 34) - 1))) * _M1
    x = (x ^ ((x >> 27) & ((1 << 37) - 1))) * _M2
    return x ^ ((x >> 31) & ((1 << 33) - 1))


_quantile_cache: dict = {}


def quantile_table(device) -> torch.Tensor:
    """N(0, 1) quantiles at (i + 0.5) / 65536, fp32, computed once on the CPU (float64 erfinv) and copied."""
    device = torch.device(device)
    t = _quantile_cache.get(device)
    if t is None:
        base = _quantile_cache.get(torch.device('cpu'))
        if base is None:
            p = (torch.arange(65536, dtype=torch.float64) + 0.5) / 65536.0
            base = (math.sqrt(2.0) * torch.erfinv(2.0 * p - 1.0)).to(torch.float32)
            _quantile_cache[torch.device('cpu')] = base
        t = _quantile_cache[device] = base.to(device)
    return t


def channel_tables(heads: int, head_dim: int, seed: int, mu: float = 0.0, s: float = 1.0, key_offset: bool = False,
                   outlier_frac: float = 0.02, outlier_scale: float = 30.0):
    """(sigma, offset) fp32 [H, D] on the CPU: sigma_c ~ LogNormal(mu, s), a fraction of channels x30,
    offset_c ~ N(0, 2) for keys (zeros otherwise)."""
    g = torch.Generator('cpu').manual_seed(int(seed))
    sigma = torch.exp(mu + s * torch.randn(heads, head_dim, generator=g))
    outlier = torch.rand(heads, head_dim, generator=g) < outlier_frac
    sigma = torch.where(outlier, sigma * outlier_scale, sigma)
    offset = 2.0 * torch.randn(heads, head_dim, generator=g) if key_offset else torch.zeros(heads, head_dim)
    return sigma.to(torch.float32), offset.to(torch.float32)


def _coords_hash(stream: int, b0: int, nb: int, H: int, s0: int, ns: int, D: int, device) -> torch.Tensor:
    """int64 [nb, H, ns, D] hash of (stream, absolute batch index, head, absolute token, dim)."""
    b = (torch.arange(b0, b0 + nb, dtype=torch.int64, device=device) * _c(0x632BE59BD9B4E019)).view(nb, 1, 1, 1)
    h = (torch.arange(H, dtype=torch.int64, device=device) * _c(0xD6E8FEB86659FD93)).view(1, H, 1, 1)
    s = (torch.arange(s0, s0 + ns, dtype=torch.int64, device=device) * _c(0xA0761D6478BD642F)).view(1, 1, ns, 1)
    d = (torch.arange(D, dtype=torch.int64, device=device) * _c(0xE7037ED1A0B428DB)).view(1, 1, 1, D)
    return _mix((b + h + s + d) ^ _c(int(stream) * 0x9E3779B97F4A7C15 + 0x1234567))


def kv_slab(stream: int, shape, sigma: torch.Tensor, offset: torch.Tensor, device='cpu', b0: int = 0, s0: int = 0,
            shift_from: int | None = None, shift_heads=None, shift_scale: float = 2.0,
            escapes=None, modulation: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 [nb, H, ns, D]: sequences b0 .. b0+nb and tokens s0 .. s0+ns of the tensor identified by
    ``stream`` (any integer: seed, layer and K/V folded together by the caller).

    shift_from / shift_heads: tokens >= shift_from of the listed heads get sigma x shift_scale.
    escapes = (left, right, p_window, p_zero): exponent fields replaced as the stress configuration asks.
    modulation: optional fp32 [ns_total, D] factor indexed by absolute token (sinusoidal magnitudes)."""
    nb, H, ns, D = shape
    device = torch.device(device)
    u = _coords_hash(stream, b0, nb, H, s0, ns, D, device)
    z = quantile_table(device)[((u >> 48) & 0xFFFF)]
    sig = sigma.to(device).view(1, H, 1, D)
    if shift_from is not None and shift_heads:
        scale = torch.ones(H, dtype=torch.float32)
        scale[list(shift_heads)] = shift_scale
        tok = torch.arange(s0, s0 + ns, device=device).view(1, 1, ns, 1)
        sig = torch.where(tok >= shift_from, sig * scale.to(device).view(1, H, 1, 1), sig)
    x = z * sig
    if modulation is not None:
        x = x * modulation.to(device)[s0:s0 + ns].view(1, 1, ns, D)
    x = (x + offset.to(device).view(1, H, 1, D)).to(torch.bfloat16)
    if escapes is not None:
        left, right, p_window, p_zero = escapes
        v = _mix(u ^ _GOLD)
        r = (v >> 32) & 0xFFFFFFFF                        # uniform 32 bits decide who escapes
        t_win = int(p_window * 4294967296.0)
        t_zero = t_win + int(p_zero * 4294967296.0)
        n_low, n_high = max(int(left), 0), max(254 - int(right), 0)
        draw = (v & 0xFFFF) % max(n_low + n_high, 1)
        new_exp = torch.where(draw < n_low, draw + 1, int(right) + 1 + (draw - n_low))
        bits = x.view(torch.int16).to(torch.int64) & 0xFFFF
        bits = torch.where(r < t_win, (bits & ~0x7F80) | (new_exp << 7), bits)
        bits = torch.where((r >= t_win) & (r < t_zero), bits & ~0x7F80, bits)
        bits = torch.where(bits >= 0x8000, bits - 0x10000, bits)
        x = bits.to(torch.int16).view(torch.bfloat16)
    return x.contiguous()


def kv_tensor(stream: int, shape, sigma, offset, device='cpu', max_elems: int = 1 << 27, **kw) -> torch.Tensor:
    """``kv_slab`` for a whole tensor, generated in batch slices so that the int64 temporaries stay
    below ``max_elems`` elements each."""
    B, H, S, D = shape
    per = max(1, max_elems // max(H * S * D, 1))
    if per >= B:
        return kv_slab(stream, shape, sigma, offset, device, **kw)
    out = torch.empty(shape, dtype=torch.bfloat16, device=device)
    b0 = kw.pop('b0', 0)
    for b in range(0, B, per):
        nb = min(per, B - b)
        out[b:b + nb] = kv_slab(stream, (nb, H, S, D), sigma, offset, device, b0=b0 + b, **kw)
    return out

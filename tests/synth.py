"""Seeded synthetic KV tensors with the value distributions of the benchmark configurations:
N(0, sigma_c) per channel with sigma_c ~ LogNormal(mu, s), 2 % outlier channels scaled x30,
an optional per-channel offset ~ N(0, 2) for keys (post-RoPE bias), and optional injected
out-of-window / zero / subnormal exponents.  Everything is generated on the CPU from a
``torch.Generator`` so the same bits appear on every machine."""
from __future__ import annotations

import torch


def kv_tensor(shape, seed: int, mu: float = 0.0, s: float = 1.0, key_offset: bool = False,
              outlier_frac: float = 0.02, outlier_scale: float = 30.0) -> torch.Tensor:
    B, H, S, D = shape
    g = torch.Generator('cpu').manual_seed(int(seed))
    sigma = torch.exp(mu + s * torch.randn(H, D, generator=g))
    outlier = torch.rand(H, D, generator=g) < outlier_frac
    sigma = torch.where(outlier, sigma * outlier_scale, sigma)
    x = torch.randn(B, H, S, D, generator=g) * sigma[None, :, None, :]
    if key_offset:
        x = x + (2.0 * torch.randn(H, D, generator=g))[None, :, None, :]
    return x.to(torch.bfloat16)


def inject_escapes(x: torch.Tensor, seed: int, left: int, right: int, p_window: float = 1e-3,
                   p_zero: float = 1e-4) -> torch.Tensor:
    """Replace the exponent field of a Bernoulli(p_window) subset by a value outside (left, right]
    drawn from [1, left] U [right+1, 254], and of a Bernoulli(p_zero) subset by 0 (zero/subnormal)."""
    g = torch.Generator('cpu').manual_seed(int(seed))
    bits = x.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    n_low = max(left, 0)
    n_high = max(254 - right, 0)
    draw = torch.randint(0, max(n_low + n_high, 1), bits.shape, generator=g)
    new_exp = torch.where(draw < n_low, draw + 1, right + 1 + (draw - n_low))
    m1 = torch.rand(bits.shape, generator=g) < p_window
    m0 = torch.rand(bits.shape, generator=g) < p_zero
    bits = torch.where(m1, (bits & ~0x7F80) | (new_exp << 7), bits)
    bits = torch.where(m0, bits & ~0x7F80, bits)
    bits = torch.where(bits >= 0x8000, bits - 0x10000, bits)
    return bits.to(torch.int16).view(torch.bfloat16).view(x.shape)


def all_bf16_patterns() -> torch.Tensor:
    """Every one of the 65 536 bf16 bit patterns, shaped [1, 4, 128, 128]."""
    v = torch.arange(65536, dtype=torch.int32)
    v = torch.where(v >= 0x8000, v - 0x10000, v).to(torch.int16)
    return v.view(torch.bfloat16).view(1, 4, 128, 128)

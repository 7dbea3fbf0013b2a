"""Seeded synthetic KV that stands in for captured KV traces.

Real KV dumps are not available, so benchmarks and parity tests use the value
distribution the benchmark configurations describe: each element is N(0,1)
scaled per channel by ``exp(N(0, 0.5))`` (one scale per layer, K-or-V, head
and dim); K has four fixed outlier channels multiplied by 8; values are
rounded to BF16 with round-to-nearest-even.  Two optional contaminations
exercise the escape and overflow paths: ``heavy`` multiplies a fraction of the
values by 64, ``junk`` replaces a fraction by uniform random finite BF16 bit
patterns.

Both a numpy form (CPU fixtures) and a torch form (large on-device workloads)
are given; they follow the same distribution but not the same random stream.
"""

from __future__ import annotations

import numpy as np
import torch

HEAD_DIM = 128
BLOCK_TOKENS = 128
K_OUTLIER_CHANNELS = (7, 42, 77, 113)
K_OUTLIER_GAIN = 8.0
HEAVY_GAIN = 64.0


def bf16_rne(x: np.ndarray) -> np.ndarray:
    """Round float32 to BF16 bit patterns (uint16), nearest-even."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


def channel_scales(seed: int, layers: int, kv_heads: int) -> np.ndarray:
    """Per-channel scales ``float32 [L, 2, H, 128]`` (K outlier channels included)."""
    rng = np.random.default_rng(seed)
    scales = np.exp(rng.normal(0.0, 0.5, (layers, 2, kv_heads, HEAD_DIM))).astype(
        np.float32
    )
    scales[:, 0, :, list(K_OUTLIER_CHANNELS)] *= K_OUTLIER_GAIN
    return scales


def kv_tokens_numpy(
    rng: np.random.Generator,
    scales: np.ndarray,
    tokens: int,
    heavy: float = 0.0,
    junk: float = 0.0,
) -> np.ndarray:
    """KV of one layer as BF16 bits ``uint16 [2, tokens, H, 128]``.

    Args:
        rng: Seeded generator.
        scales: ``[2, H, 128]`` channel scales of the layer.
        tokens: Tokens to draw.
        heavy: Fraction of values multiplied by 64.
        junk: Fraction of values replaced by random finite BF16 bit patterns.
    """
    heads = scales.shape[1]
    x = rng.standard_normal((2, tokens, heads, HEAD_DIM), dtype=np.float32)
    x *= scales[:, None]
    if heavy:
        x[rng.random(x.shape) < heavy] *= HEAVY_GAIN
    bits = bf16_rne(x)
    if junk:
        mask = rng.random(bits.shape) < junk
        patt = rng.integers(0, 1 << 16, size=int(mask.sum()), dtype=np.uint16)
        # Keep them finite: an all-ones exponent (0x7F80) is cleared to 0x7F00.
        inf = (patt & 0x7F80) == 0x7F80
        patt[inf] &= 0xFF7F
        bits[mask] = patt
    return bits


def kv_tokens_torch(
    gen: torch.Generator,
    scales: torch.Tensor,
    tokens: int,
    heavy: float = 0.0,
    junk: float = 0.0,
) -> torch.Tensor:
    """KV of one layer as BF16 ``[2, tokens, H, 128]`` on ``scales.device``.

    Args:
        gen: Seeded generator on the same device as ``scales``.
        scales: float32 ``[2, H, 128]``.
        tokens: Tokens to draw.
        heavy: Fraction of values multiplied by 64.
        junk: Fraction of values replaced by random finite BF16 bit patterns.
    """
    dev = scales.device
    heads = scales.shape[1]
    x = torch.randn((2, tokens, heads, HEAD_DIM), generator=gen, device=dev)
    x *= scales[:, None]
    if heavy:
        hit = torch.rand(x.shape, generator=gen, device=dev) < heavy
        x = torch.where(hit, x * HEAVY_GAIN, x)
    out = x.to(torch.bfloat16)
    if junk:
        hit = torch.rand(out.shape, generator=gen, device=dev) < junk
        patt = torch.randint(0, 1 << 16, out.shape, generator=gen, device=dev, dtype=torch.int32)
        patt = torch.where((patt & 0x7F80) == 0x7F80, patt & 0xFF7F, patt)
        patt = torch.where(patt >= 1 << 15, patt - (1 << 16), patt).to(torch.int16)
        out = torch.where(hit, patt.view(torch.bfloat16), out)
    return out


def calibration_dump(
    seed: int, scales: np.ndarray, samples: int = 64, heavy: float = 0.0, junk: float = 0.0
) -> np.ndarray:
    """Calibration pages ``uint16 [S, L, 2, 128, H, 128]`` drawn like the KV."""
    rng = np.random.default_rng(seed)
    layers, _, heads, _ = scales.shape
    dump = np.empty((samples, layers, 2, BLOCK_TOKENS, heads, HEAD_DIM), np.uint16)
    for layer in range(layers):
        kv = kv_tokens_numpy(rng, scales[layer], samples * BLOCK_TOKENS, heavy, junk)
        dump[:, layer] = kv.reshape(2, samples, BLOCK_TOKENS, heads, HEAD_DIM).transpose(
            1, 0, 2, 3, 4
        )
    return dump


__all__ = [
    "bf16_rne",
    "calibration_dump",
    "channel_scales",
    "kv_tokens_numpy",
    "kv_tokens_torch",
]

"""per_channel_cast (reference: tile_kernels/quant/per_channel_cast_kernel.py:8-28): the plain-input case of the
fused per-channel cast, kept as its own entry point."""
import torch

from .per_channel_cast_fused_kernel import per_channel_cast_fused
from .types import QuantTensor

_TOKENS_PER_SCALE = 128


def per_channel_cast(x: torch.Tensor, fmt: str, num_per_tokens: int, round_sf: bool = False) -> QuantTensor:
    """FP8 e4m3 cast with one scale per (128 tokens x 1 channel).

    x is a contiguous (num_tokens, hidden) matrix with num_tokens % 128 == 0 and hidden % 64 == 0.
    Returns (out, out_sf): float8_e4m3fn (num_tokens, hidden) and float32 (num_tokens // 128, hidden); with
    `round_sf` the scales are powers of two."""
    assert fmt == 'e4m3', 'per_channel_cast produces FP8 e4m3 only'
    assert num_per_tokens == _TOKENS_PER_SCALE, 'one scale covers 128 tokens'
    assert x.dim() == 2 and x.is_contiguous(), 'x must be a contiguous matrix'
    assert x.size(0) % _TOKENS_PER_SCALE == 0 and x.size(1) % 64 == 0, 'whole 128-token blocks, hidden % 64 == 0'
    return per_channel_cast_fused(x, fmt, _TOKENS_PER_SCALE, round_sf)

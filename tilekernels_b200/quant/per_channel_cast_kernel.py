"""per_channel_cast (reference: tile_kernels/quant/per_channel_cast_kernel.py:8-28)."""
import torch

from .per_channel_cast_fused_kernel import per_channel_cast_fused
from .types import QuantTensor


def per_channel_cast(x: torch.Tensor, fmt: str, num_per_tokens: int, round_sf: bool = False) -> QuantTensor:
    """Cast a contiguous matrix to FP8 e4m3 with one scale per (128 tokens x 1 channel).

    Returns (out, out_sf): float8_e4m3fn (num_tokens, hidden) and float32 (num_tokens / 128, hidden)."""
    assert x.is_contiguous() and x.dim() == 2
    assert fmt == 'e4m3'
    num_tokens, hidden = x.shape
    assert num_tokens % 128 == 0 and hidden % 64 == 0
    assert num_per_tokens == 128
    return per_channel_cast_fused(x, 'e4m3', num_per_tokens=num_per_tokens, round_sf=round_sf)

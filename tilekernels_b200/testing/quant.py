import torch

from ..utils import align, ceil_div


def clear_unused_sf(sf: torch.Tensor, hidden: int, num_per_channels: int) -> torch.Tensor:
    """Flatten packed scales to bytes, one row of align(groups, 4) per token block, and zero the padding
    bytes beyond the last group (same contract as the reference's tile_kernels/testing/quant.py:6-21)."""
    groups = ceil_div(hidden, num_per_channels)
    dense = torch.empty(sf.shape, dtype=sf.dtype, device=sf.device)
    dense.copy_(sf)
    flat = dense.flatten().view(torch.uint8).view(-1, align(groups, 4))
    flat[:, groups:] = 0
    return flat

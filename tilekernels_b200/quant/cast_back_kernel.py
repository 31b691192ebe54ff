"""cast_back / per_token_cast_back (reference: tile_kernels/quant/cast_back_kernel.py:77-143)."""
from typing import Optional

import torch

from .. import _lib
from .cast_back_e5m6_kernel import cast_back_e5m6, launch_cast_back
from .common import get_cast_input_and_config, get_logical_hidden
from .types import QuantTensor


def cast_back(
    x: QuantTensor,
    fmt: str,
    x_block_size: tuple[int, int],
    x_special_fmt: Optional[str] = None,
) -> torch.Tensor:
    """Dequantise an FP8 / FP4 (or, with x_special_fmt='e5m6', packed E5M6) tensor to bfloat16 or float32.

    Args:
        x: (data, scales); data float8_e4m3fn or int8 (two FP4 per byte); scales in any layout the casts produce.
        fmt: 'bf16' or 'fp32'.
        x_block_size: scale block (tokens, channels).
    """
    assert fmt in ('bf16', 'fp32')
    data, x_sf = x
    if x_special_fmt == 'e5m6':
        assert data.dtype == torch.uint8
        return cast_back_e5m6((data, x_sf), fmt, x_block_size)
    assert x_special_fmt is None, f'Unsupported special format: {x_special_fmt}'

    num_tokens, hidden = data.shape
    assert x_sf.dim() == 2
    assert x_sf.dtype in (torch.int32, torch.float32)
    hidden = get_logical_hidden(hidden, data.dtype)
    assert hidden % 64 == 0
    assert data.dtype in (torch.float8_e4m3fn, torch.int8) and data.is_contiguous() and data.is_cuda

    data, x_sf, in_config = get_cast_input_and_config((data, x_sf), tuple(x_block_size))
    in_fmt = _lib.FMT_E4M3 if data.dtype == torch.float8_e4m3fn else _lib.FMT_E2M1
    return launch_cast_back(data, in_fmt, x_sf, in_config, num_tokens, hidden, fmt)


def per_token_cast_back(
    x: QuantTensor,
    fmt: str,
    num_per_channels: int,
    x_special_fmt: Optional[str] = None,
) -> torch.Tensor:
    """cast_back with one scale per (1 x num_per_channels) group of a token."""
    return cast_back(x, fmt, (1, num_per_channels), x_special_fmt=x_special_fmt)

"""per_token_cast and its two variants (reference: tile_kernels/quant/per_token_cast_kernel.py:159-302)."""
from typing import Optional, Union

import torch

from .. import _lib
from .common import (device_guard, DTYPE_TO_ENUM, FMT_TO_ENUM, alloc_scaling_factors, cast_epilogue, current_stream_ptr,
                     get_cast_input_and_config, get_cast_output_config, get_logical_hidden, get_physical_hidden)
from .per_token_cast_to_e5m6_kernel import per_token_cast_to_e5m6
from .types import QuantTensor


def per_token_cast_impl(
    x: torch.Tensor,
    fmt: str,
    num_per_channels: int,
    x_block_size: Optional[tuple[int, int]] = None,
    use_tma_aligned_col_major_sf: bool = False,
    round_sf: bool = False,
    use_packed_ue8m0: bool = False,
    sf_only: bool = False,
    sf: Optional[torch.Tensor] = None,
) -> Union[torch.Tensor, QuantTensor]:
    assert fmt in ('e5m6', 'e4m3', 'e2m1')
    if fmt == 'e5m6':
        assert x_block_size is None
        assert not sf_only
        assert sf is None
        return per_token_cast_to_e5m6(x, num_per_channels, use_tma_aligned_col_major_sf, round_sf, use_packed_ue8m0)

    x, x_sf, in_config = get_cast_input_and_config(x, x_block_size)
    out_config = get_cast_output_config(fmt, (1, num_per_channels), use_tma_aligned_col_major_sf, round_sf, use_packed_ue8m0)

    assert x.dim() == 2 and x.is_cuda and (x.shape[1] == 0 or x.stride(1) == 1)
    num_tokens, hidden = x.shape
    hidden = get_logical_hidden(hidden, x.dtype)
    assert num_per_channels in (16, 32, 64, 128) or (num_per_channels == hidden and hidden % 64 == 0)
    if num_per_channels == hidden and num_per_channels not in (16, 32, 64, 128):
        assert not sf_only and sf is None  # one scale per token has no sf-only / cast-only form
        assert not in_config.with_sf
    if in_config.with_sf:
        assert not sf_only and sf is None
        assert num_per_channels in (16, 32, 64, 128) and in_config.sf_block[1] % 16 == 0

    flags = out_config.flags
    if sf_only:
        flags |= _lib.SF_ONLY
    if sf is not None:
        assert not use_tma_aligned_col_major_sf and not use_packed_ue8m0
        assert sf.dtype == torch.float32 and sf.dim() == 2 and sf.stride(1) == 1
        assert tuple(sf.shape) == (num_tokens, -(-hidden // num_per_channels))
        flags |= _lib.CAST_ONLY

    out = torch.empty((num_tokens, get_physical_hidden(hidden, out_config.torch_dtype)), dtype=out_config.torch_dtype,
                      device=x.device)
    out_sf = sf if sf is not None else alloc_scaling_factors((num_tokens, hidden), out_config=out_config, device=x.device)
    if num_tokens > 0:
        with device_guard(x.device):
            if in_config.with_sf:
                rc = _lib.lib().tkq_per_token_cast_quantized(
                    x.data_ptr(), _lib.FMT_E4M3 if x.dtype == torch.float8_e4m3fn else _lib.FMT_E2M1, x_sf.data_ptr(),
                    in_config.flags, x_sf.stride(0), in_config.sf_block[0], in_config.sf_block[1], num_tokens, hidden,
                    get_logical_hidden(x.stride(0), x.dtype), FMT_TO_ENUM[fmt], num_per_channels, flags, out.data_ptr(),
                    out_sf.data_ptr(), out_sf.stride(0), current_stream_ptr(x.device))
                _lib.check(rc, 'tkq_per_token_cast_quantized')
            else:
                rc = _lib.lib().tkq_per_token_cast(
                    x.data_ptr(), DTYPE_TO_ENUM[x.dtype], num_tokens, hidden, x.stride(0), FMT_TO_ENUM[fmt], num_per_channels,
                    flags, out.data_ptr(), out_sf.data_ptr(), out_sf.stride(0), current_stream_ptr(x.device))
                _lib.check(rc, 'tkq_per_token_cast')

    out_sf = cast_epilogue(out_sf, num_tokens, hidden, out_config)
    if sf_only:
        return out_sf
    if sf is not None:
        return out
    return out, out_sf


def per_token_cast(
    x: torch.Tensor,
    fmt: str,
    num_per_channels: int,
    x_block_size: Optional[tuple[int, int]] = None,
    use_tma_aligned_col_major_sf: bool = False,
    round_sf: bool = False,
    use_packed_ue8m0: bool = False,
) -> QuantTensor:
    """Cast a matrix to FP8 / FP4 / E5M6 with one scale per (1 x num_per_channels) group of a token.

    Args:
        x: 2-D CUDA tensor (num_tokens, hidden), bfloat16 or float32, rows may be strided; or an already
            quantized pair (data, scales) with data float8_e4m3fn or int8 (two FP4 per byte).
        fmt: 'e4m3', 'e2m1' or 'e5m6'.
        num_per_channels: 16, 32, 64, 128 or hidden ('e5m6': hidden).
        x_block_size: scale block (rows, channels) of an already quantized input, e.g. (128, 128) or (32, 32).
        use_tma_aligned_col_major_sf: column-major scales, token dimension padded to 16 bytes.
        round_sf: round scales up to powers of two.
        use_packed_ue8m0: store scales as exponent bytes, four per int32.

    Returns:
        (out, out_sf): quantized data and scales, dtypes/shapes/strides as in the reference.
    """
    return per_token_cast_impl(x, fmt, num_per_channels, x_block_size, use_tma_aligned_col_major_sf, round_sf, use_packed_ue8m0)


def per_token_cast_with_sf_only(
    x: torch.Tensor,
    fmt: str,
    num_per_channels: int,
    x_block_size: Optional[tuple[int, int]] = None,
    use_tma_aligned_col_major_sf: bool = False,
    round_sf: bool = False,
    use_packed_ue8m0: bool = False,
) -> torch.Tensor:
    """As per_token_cast, but only the scales are computed and returned."""
    return per_token_cast_impl(x, fmt, num_per_channels, x_block_size, use_tma_aligned_col_major_sf, round_sf, use_packed_ue8m0,
                               sf_only=True)


def per_token_cast_with_precomputed_sf(
    x: torch.Tensor,
    fmt: str,
    num_per_channels: int,
    sf: torch.Tensor,
    x_block_size: Optional[tuple[int, int]] = None,
    use_tma_aligned_col_major_sf: bool = False,
    round_sf: bool = False,
    use_packed_ue8m0: bool = False,
) -> torch.Tensor:
    """As per_token_cast, but with the given row-major fp32 scales `sf`; returns only the data."""
    return per_token_cast_impl(x, fmt, num_per_channels, x_block_size, use_tma_aligned_col_major_sf, round_sf, use_packed_ue8m0,
                               sf_only=False, sf=sf)

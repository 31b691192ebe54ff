"""per_block_cast and its two variants (reference: tile_kernels/quant/per_block_cast_kernel.py:141-276)."""
from typing import Optional, Union

import torch

from .. import _lib
from ..utils import ceil_div
from .common import (device_guard, DTYPE_TO_ENUM, FMT_TO_ENUM, alloc_scaling_factors, cast_epilogue, current_stream_ptr,
                     get_cast_input_and_config, get_cast_output_config)
from .types import QuantTensor


def per_block_cast_impl(
    x: torch.Tensor,
    fmt: str,
    block_size: tuple[int, int],
    use_tma_aligned_col_major_sf: bool = False,
    round_sf: bool = False,
    use_packed_ue8m0: bool = False,
    sf_only: bool = False,
    sf: Optional[torch.Tensor] = None,
) -> Union[torch.Tensor, QuantTensor]:
    assert x.is_contiguous() and x.dim() == 2 and x.is_cuda
    num_tokens, hidden = x.shape
    assert hidden % 64 == 0
    assert fmt in ('e4m3', 'e2m1')
    assert block_size[0] in (32, 128) and block_size[1] in (32, 128)
    if sf is not None:
        assert not sf_only and not use_tma_aligned_col_major_sf and not use_packed_ue8m0
        assert sf.dtype == torch.float32 and sf.dim() == 2 and sf.stride(1) == 1
        assert tuple(sf.shape) == (ceil_div(num_tokens, block_size[0]), ceil_div(hidden, block_size[1]))

    x, _, _ = get_cast_input_and_config(x, None)
    out_config = get_cast_output_config(fmt, tuple(block_size), use_tma_aligned_col_major_sf, round_sf, use_packed_ue8m0)
    flags = out_config.flags | (_lib.SF_ONLY if sf_only else 0) | (_lib.CAST_ONLY if sf is not None else 0)

    out = torch.empty((num_tokens, hidden if fmt == 'e4m3' else hidden // 2), dtype=out_config.torch_dtype, device=x.device)
    out_sf = sf if sf is not None else alloc_scaling_factors((num_tokens, hidden), out_config=out_config, device=x.device)
    if num_tokens > 0:
        with device_guard(x.device):
            rc = _lib.lib().tkq_per_block_cast(
                x.data_ptr(), DTYPE_TO_ENUM[x.dtype], num_tokens, hidden, FMT_TO_ENUM[fmt], block_size[0], block_size[1],
                flags, out.data_ptr(), out_sf.data_ptr(), out_sf.stride(0), current_stream_ptr(x.device))
        _lib.check(rc, 'tkq_per_block_cast')

    out_sf = cast_epilogue(out_sf, num_tokens, hidden, out_config)
    if sf_only:
        return out_sf
    if sf is not None:
        return out
    return out, out_sf


def per_block_cast(
    x: torch.Tensor,
    fmt: str,
    block_size: tuple[int, int],
    use_tma_aligned_col_major_sf: bool = False,
    round_sf: bool = False,
    use_packed_ue8m0: bool = False,
) -> QuantTensor:
    """Cast a contiguous matrix to FP8 / FP4 with one scale per (block_m x block_k) block (32 or 128 each).

    Returns (out, out_sf) with the reference's dtypes, shapes and strides."""
    return per_block_cast_impl(x, fmt, block_size, use_tma_aligned_col_major_sf, round_sf, use_packed_ue8m0)


def per_block_cast_with_sf_only(
    x: torch.Tensor,
    fmt: str,
    block_size: tuple[int, int],
    use_tma_aligned_col_major_sf: bool = False,
    round_sf: bool = False,
    use_packed_ue8m0: bool = False,
) -> torch.Tensor:
    """As per_block_cast, but only the scales are computed and returned."""
    return per_block_cast_impl(x, fmt, block_size, use_tma_aligned_col_major_sf, round_sf, use_packed_ue8m0, sf_only=True)


def per_block_cast_with_precomputed_sf(
    x: torch.Tensor,
    fmt: str,
    block_size: tuple[int, int],
    sf: torch.Tensor,
    use_tma_aligned_col_major_sf: bool = False,
    round_sf: bool = False,
    use_packed_ue8m0: bool = False,
) -> torch.Tensor:
    """As per_block_cast, but with the given row-major fp32 scales `sf`; returns only the data."""
    return per_block_cast_impl(x, fmt, block_size, use_tma_aligned_col_major_sf, round_sf, use_packed_ue8m0, sf_only=False, sf=sf)

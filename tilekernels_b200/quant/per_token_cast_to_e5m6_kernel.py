"""per_token_cast_to_e5m6 (reference: tile_kernels/quant/per_token_cast_to_e5m6_kernel.py:159-215)."""
import torch

from .. import _lib
from .common import (device_guard, DTYPE_TO_ENUM, alloc_scaling_factors, cast_epilogue, current_stream_ptr, get_cast_input_and_config,
                     get_cast_output_config)
from .types import QuantTensor


def per_token_cast_to_e5m6(
    x: torch.Tensor,
    num_per_channels: int,
    use_tma_aligned_col_major_sf: bool = False,
    round_sf: bool = False,
    use_packed_ue8m0: bool = False,
) -> QuantTensor:
    """Cast a matrix to E5M6 (1 sign, 5 exponent, 6 mantissa bits; 8 values in 3 uint32) with one scale per token.

    Args:
        x: 2-D CUDA tensor (num_tokens, hidden), bfloat16 or float32, hidden % 8 == 0.
        num_per_channels: must equal hidden.

    Returns:
        (out, out_sf): uint8 (num_tokens, hidden * 3 // 2) and the scales.
    """
    assert x.dtype == torch.bfloat16 or x.dtype == torch.float32
    assert x.dim() == 2 and x.is_cuda and (x.shape[1] == 0 or x.stride(1) == 1)
    num_tokens, hidden = x.shape
    assert num_per_channels == hidden
    assert hidden % 8 == 0

    x, _, _ = get_cast_input_and_config(x, None)
    out_config = get_cast_output_config('e5m6', (1, num_per_channels), use_tma_aligned_col_major_sf, round_sf, use_packed_ue8m0, 1e-4)

    out = torch.empty((num_tokens, hidden // 8 * 3), dtype=torch.uint32, device=x.device)
    out_sf = alloc_scaling_factors((num_tokens, hidden), out_config=out_config, device=x.device)
    if num_tokens > 0:
        with device_guard(x.device):
            rc = _lib.lib().tkq_per_token_cast_e5m6(
                x.data_ptr(), DTYPE_TO_ENUM[x.dtype], num_tokens, hidden, x.stride(0), out_config.flags, out.data_ptr(),
                out_sf.data_ptr(), out_sf.stride(0), current_stream_ptr(x.device))
        _lib.check(rc, 'tkq_per_token_cast_e5m6')

    out = out.view(torch.uint8)
    out_sf = cast_epilogue(out_sf, num_tokens, hidden, out_config)
    return out, out_sf

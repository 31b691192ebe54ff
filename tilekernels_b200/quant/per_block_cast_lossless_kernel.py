"""per_block_cast_lossless (reference: tile_kernels/quant/per_block_cast_lossless_kernel.py:154-209)."""
import torch

from .. import _lib
from .common import (device_guard, alloc_scaling_factors, cast_epilogue, current_stream_ptr, get_cast_input_and_config, get_cast_output_config,
                     get_logical_hidden)
from .types import QuantTensor


def per_block_cast_lossless(
    x: QuantTensor,
    fmt: str,
    x_block_size: tuple[int, int],
    out_block_size: tuple[int, int],
    use_tma_aligned_col_major_sf: bool = False,
    round_sf: bool = False,
    use_packed_ue8m0: bool = False,
) -> QuantTensor:
    """Re-quantize an FP4 (e2m1, power-of-two scales) tensor to FP8 e4m3 with new scale blocks without loss:
    the output scale of a block is the largest input scale inside it divided by 2^6.

    Args:
        x: (data int8 with two FP4 per byte, scales in any layout the casts produce).
        fmt: 'e4m3'.
        x_block_size / out_block_size: (tokens, channels) per scale; output (1|32|128) x (32|128).

    Returns:
        (out, out_sf): float8_e4m3fn (num_tokens, hidden) and the scales (powers of two).
    """
    data, x_sf, in_config = get_cast_input_and_config(x, tuple(x_block_size))
    assert fmt == 'e4m3' and data.dtype == torch.int8, 'lossless cast only supports e2m1 -> e4m3 input'
    assert data.dim() == 2 and data.is_cuda and data.stride(1) == 1
    num_tokens, hidden = data.shape
    hidden = get_logical_hidden(hidden, data.dtype)
    assert hidden % 32 == 0
    assert out_block_size[0] % x_block_size[0] == 0 and out_block_size[1] % x_block_size[1] == 0

    out_config = get_cast_output_config(fmt, tuple(out_block_size), use_tma_aligned_col_major_sf, round_sf, use_packed_ue8m0)
    out = torch.empty((num_tokens, hidden), dtype=out_config.torch_dtype, device=data.device)
    out_sf = alloc_scaling_factors((num_tokens, hidden), out_config=out_config, device=data.device)
    if num_tokens > 0:
        with device_guard(data.device):
            rc = _lib.lib().tkq_per_block_cast_lossless(
                data.data_ptr(), x_sf.data_ptr(), in_config.flags, x_sf.stride(0), x_block_size[0], x_block_size[1], num_tokens,
                hidden, get_logical_hidden(data.stride(0), data.dtype), out_block_size[0], out_block_size[1],
                out_config.flags & ~_lib.ROUND_SF, out.data_ptr(), out_sf.data_ptr(), out_sf.stride(0), current_stream_ptr(data.device))
        _lib.check(rc, 'tkq_per_block_cast_lossless')
    return out, cast_epilogue(out_sf, num_tokens, hidden, out_config)

"""per_channel_cast_fused (reference: tile_kernels/quant/per_channel_cast_fused_kernel.py:137-203)."""
from typing import Optional, Union

import torch

from .. import _lib
from ..utils import ceil_div
from .common import DTYPE_TO_ENUM, current_stream_ptr, device_guard
from .types import QuantTensor

_IN_FP8 = 2  # input kind of tkq_per_channel_cast_fused next to the bf16 / fp32 enums


def per_channel_cast_fused(
    x: Union[torch.Tensor, QuantTensor],
    fmt: str,
    num_per_tokens: int,
    round_sf: bool = False,
    num_per_channels: Optional[int] = None,
    pos_to_token: Optional[torch.Tensor] = None,
) -> QuantTensor:
    """Cast a matrix to FP8 e4m3 with one scale per (128 tokens x 1 channel), optionally fusing a rescale of
    FP8 input and a row gather.

    Args:
        x: contiguous CUDA tensor (num_tokens, hidden), bfloat16 / float32, or a pair (float8_e4m3fn data,
            float32 scales of shape (num_tokens, hidden / 128)) that is rescaled on the fly.
        fmt: 'e4m3'.
        num_per_tokens: 128.
        round_sf: round scales up to powers of two.
        num_per_channels: 128 when x is a pair, else None.
        pos_to_token: optional int32 (num_tokens_out,), a multiple of 16 long: output row i is input row
            pos_to_token[i]; a negative entry gives a row of zeros.

    Returns:
        (out, out_sf): float8_e4m3fn (num_tokens_out, hidden) and float32 (ceil(num_tokens_out / 128), hidden).
    """
    x_sf = None
    if isinstance(x, tuple):
        assert num_per_channels is not None
        x, x_sf = x
    else:
        assert num_per_channels is None
    assert fmt == 'e4m3'
    assert x.dim() == 2 and x.is_contiguous() and x.is_cuda
    num_tokens, hidden = x.shape
    num_tokens_out = num_tokens

    if pos_to_token is not None:
        assert pos_to_token.dim() == 1 and pos_to_token.is_contiguous()
        assert pos_to_token.dtype == torch.int32
        num_tokens_out = pos_to_token.size(0)
        assert num_tokens_out % 16 == 0  # alignment of expanded token counts
    else:
        assert num_tokens_out % 128 == 0
    assert num_per_tokens == 128
    assert hidden % 64 == 0
    if x_sf is not None:
        assert num_per_channels == 128
        assert x.dtype == torch.float8_e4m3fn
        assert x_sf.dim() == 2 and x_sf.is_contiguous() and x_sf.dtype == torch.float32
        assert x_sf.size(0) == num_tokens and x_sf.size(1) * 128 == hidden
        in_kind = _IN_FP8
    else:
        assert x.dtype in (torch.bfloat16, torch.float32)
        in_kind = DTYPE_TO_ENUM[x.dtype]

    out = torch.empty((num_tokens_out, hidden), dtype=torch.float8_e4m3fn, device=x.device)
    out_sf = torch.empty((ceil_div(num_tokens_out, num_per_tokens), hidden), dtype=torch.float32, device=x.device)
    if num_tokens_out > 0:
        flags = _lib.ROUND_SF if round_sf else 0
        with device_guard(x.device):
            if x_sf is None and pos_to_token is None:  # rectangular input: the TMA tile pipeline
                rc = _lib.lib().tkq_per_channel_cast(x.data_ptr(), in_kind, num_tokens, hidden, flags, out.data_ptr(),
                                                     out_sf.data_ptr(), current_stream_ptr(x.device))
                _lib.check(rc, 'tkq_per_channel_cast')
            else:
                rc = _lib.lib().tkq_per_channel_cast_fused(
                    x.data_ptr(), in_kind, None if x_sf is None else x_sf.data_ptr(),
                    None if pos_to_token is None else pos_to_token.data_ptr(), num_tokens, num_tokens_out, hidden, flags,
                    out.data_ptr(), out_sf.data_ptr(), current_stream_ptr(x.device))
                _lib.check(rc, 'tkq_per_channel_cast_fused')
    return out, out_sf

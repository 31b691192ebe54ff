"""cast_back_e5m6 (reference: tile_kernels/quant/cast_back_e5m6_kernel.py:134-176) and the launch shared with cast_back."""
import torch

from .. import _lib
from .common import CastInputConfig, current_stream_ptr, get_cast_input_and_config, device_guard
from .types import QuantTensor


def launch_cast_back(data: torch.Tensor, in_fmt: int, x_sf: torch.Tensor, in_config: CastInputConfig, num_tokens: int,
                     hidden: int, fmt: str) -> torch.Tensor:
    """Allocate the output and enqueue tkq_cast_back; `x_sf` is the scale storage get_cast_input_and_config returns."""
    out = torch.empty((num_tokens, hidden), dtype=torch.bfloat16 if fmt == 'bf16' else torch.float32, device=data.device)
    if num_tokens > 0:
        with device_guard(data.device):
            rc = _lib.lib().tkq_cast_back(data.data_ptr(), in_fmt, x_sf.data_ptr(), in_config.flags, x_sf.stride(0),
                                          in_config.sf_block[0], in_config.sf_block[1], num_tokens, hidden,
                                          _lib.DT_BF16 if fmt == 'bf16' else _lib.DT_FP32, out.data_ptr(),
                                          current_stream_ptr(data.device))
        _lib.check(rc, 'tkq_cast_back')
    return out


def cast_back_e5m6(
    x: QuantTensor,
    fmt: str,
    x_block_size: tuple[int, int],
) -> torch.Tensor:
    """Dequantise a packed E5M6 tensor (uint8, hidden * 3 / 2 bytes per token) to bfloat16 or float32."""
    assert fmt in ('bf16', 'fp32')
    data, x_sf = x
    num_tokens = data.size(0)
    assert data.dim() == 2 and data.is_contiguous() and data.is_cuda
    assert x_sf.dim() == 2
    assert x_sf.dtype in (torch.int32, torch.float32)
    assert data.dtype == torch.uint8
    hidden = data.size(1) * 2 // 3
    # the dequantisation kernel works on 16 values per lane (the cast itself accepts hidden % 8 == 0)
    assert hidden % 16 == 0, 'cast_back_e5m6 needs hidden % 16 == 0'
    data, x_sf, in_config = get_cast_input_and_config((data, x_sf), tuple(x_block_size))
    return launch_cast_back(data, _lib.FMT_E5M6, x_sf, in_config, num_tokens, hidden, fmt)

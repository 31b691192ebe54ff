"""swiglu_backward_and_per_token_cast
(reference: tile_kernels/quant/swiglu_backward_and_per_token_cast_kernel.py:157-238)."""
from typing import Optional

import torch

from .. import _lib
from .common import current_stream_ptr, device_guard
from .types import QuantTensor


def swiglu_backward_and_per_token_cast(
    x: QuantTensor,
    grad_out: torch.Tensor,
    weight: torch.Tensor,
    pos_to_token_topk: torch.Tensor,
    token_topk_to_pos: torch.Tensor,
    num_per_channels: int,
    round_sf: bool = False,
    swiglu_clamp_value: Optional[float] = None,
) -> tuple[torch.Tensor, QuantTensor, torch.Tensor, torch.Tensor]:
    """SwiGLU backward with the per-token FP8 cast of the input gradient, in one kernel.

    Args:
        x: the forward input as (data, sf): data (num_expand_tokens, 2 * hidden) float8_e4m3fn, sf
            (num_expand_tokens, 2 * hidden // num_per_channels) float32.
        grad_out: bfloat16 gradient of the weighted activation, (num_expand_tokens, hidden).
        weight: top-k routing weights (num_tokens, num_topk), float32.
        pos_to_token_topk: int32 per expanded position, the flat (token, k) index or a negative value.
        token_topk_to_pos: int32 (num_tokens, num_topk), the expanded position or -1.
        num_per_channels: 32 or 128.
        round_sf: power-of-two scales for the quantised gradient.
        swiglu_clamp_value: the clamp the forward pass used, or None.

    Returns:
        (out, (x_grad_fp8, x_grad_fp8_sf), x_grad, weight_grad): the weighted activation (bfloat16), the
        quantised input gradient with its float32 scales, the bfloat16 input gradient and the float32
        gradient of the routing weights.
    """
    assert num_per_channels in (32, 128)
    x, x_sf = x

    assert x.dtype == torch.float8_e4m3fn
    assert (x.dim() == 2 or x.dim() == 3) and x.is_contiguous() and x.is_cuda
    assert x_sf.dim() == 2 and x_sf.is_contiguous() and x_sf.dtype == torch.float32
    assert weight.dim() == 2 and weight.is_contiguous() and weight.dtype == torch.float32
    assert pos_to_token_topk.dim() == 1 and pos_to_token_topk.is_contiguous() and pos_to_token_topk.dtype == torch.int32
    assert token_topk_to_pos.dim() == 2 and token_topk_to_pos.is_contiguous() and token_topk_to_pos.dtype == torch.int32
    assert grad_out.dtype == torch.bfloat16 and grad_out.is_contiguous()

    assert x.size(-1) % (2 * num_per_channels) == 0
    hidden = x.size(-1) // 2

    x = x.view(-1, hidden * 2)
    grad_out = grad_out.view(-1, hidden)
    num_expand_tokens = x.size(0)
    num_tokens, num_topk = token_topk_to_pos.shape

    assert x_sf.shape == (num_expand_tokens, 2 * hidden // num_per_channels)
    assert grad_out.shape == (num_expand_tokens, hidden)
    assert weight.shape == (num_tokens, num_topk)
    assert pos_to_token_topk.shape == (num_expand_tokens, )

    out = torch.empty((num_expand_tokens, hidden), dtype=grad_out.dtype, device=grad_out.device)
    x_grad_fp8 = torch.empty((num_expand_tokens, hidden * 2), dtype=x.dtype, device=x.device)
    x_grad_fp8_sf = torch.empty((num_expand_tokens, 2 * hidden // num_per_channels), dtype=torch.float32, device=x.device)
    x_grad = torch.empty((num_expand_tokens, hidden * 2), dtype=grad_out.dtype, device=grad_out.device)
    weight_grad = torch.empty((num_tokens, num_topk), dtype=torch.float32, device=x.device)

    if num_expand_tokens > 0:
        with device_guard(x.device):
            _lib.check(_lib.lib().tkq_swiglu_backward_and_per_token_cast(
                x.data_ptr(), x_sf.data_ptr(), grad_out.data_ptr(), weight.data_ptr(), pos_to_token_topk.data_ptr(),
                token_topk_to_pos.data_ptr(), num_expand_tokens, hidden, num_tokens, num_topk, num_per_channels,
                -1.0 if swiglu_clamp_value is None else float(swiglu_clamp_value), _lib.ROUND_SF if round_sf else 0,
                out.data_ptr(), x_grad_fp8.data_ptr(), x_grad_fp8_sf.data_ptr(), x_grad.data_ptr(), weight_grad.data_ptr(),
                current_stream_ptr(x.device)), 'swiglu_backward_and_per_token_cast')

    return out, (x_grad_fp8, x_grad_fp8_sf), x_grad, weight_grad

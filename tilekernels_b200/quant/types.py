import torch

# (quantized data, scale factors) -- same alias as the reference's tile_kernels/quant/types.py:3
QuantTensor = tuple[torch.Tensor, torch.Tensor]

import torch
import torch.nn as nn


class MorphoModule(nn.Module):
    """Holds the structuring element of a morphological layer: zeros of shape
    (out_channels, in_channels, K_h, K_w), or (channels, 1, K_h, K_w) for the 'identity' merge, under the
    parameter name `weight` (reference: morphocore/nn/morpho_module.py:6-22), so state dicts interchange."""

    def __init__(self, in_channels: int, out_channels: int, kernel_shape: tuple, channel_merge_mode: str = "sum",
                 padding_mode: str = "replicate", dtype: torch.dtype = torch.float32, padding_value: float = 0.0):
        super().__init__()
        if channel_merge_mode == "identity":
            if in_channels != out_channels:
                raise ValueError("For 'identity' channel_merge_mode, in_channels must be equal to out_channels.")
            self.weight = nn.Parameter(torch.zeros((out_channels, 1, *kernel_shape), dtype=dtype))
        else:
            self.weight = nn.Parameter(torch.zeros((out_channels, in_channels, *kernel_shape), dtype=dtype))
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.channel_merge_mode = channel_merge_mode
        self.padding_mode = padding_mode
        self.padding_value = padding_value

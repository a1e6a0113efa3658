import torch
import torch.nn as nn

from .morpho_module import MorphoModule


class AlphaModule(MorphoModule):
    """MorphoModule plus the learnable `alpha` of the smooth operators: (out_channels, in_channels), or
    (channels, 1) for the 'identity' merge (reference: morphocore/nn/alpha_module.py:7-19)."""

    def __init__(self, in_channel: int, out_channel: int, kernel_shape: tuple, channel_merge_mode: str = "sum",
                 init_alpha: float = 0.0, dtype: torch.dtype = torch.float32):
        super().__init__(in_channel, out_channel, kernel_shape, channel_merge_mode)
        if channel_merge_mode == 'identity':
            self.alpha = nn.Parameter(torch.full((out_channel, 1), init_alpha, dtype=dtype))
        else:
            self.alpha = nn.Parameter(torch.full((out_channel, in_channel), init_alpha, dtype=dtype))

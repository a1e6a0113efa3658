import torch

from morphocore_b200.functional import erosion
from .morpho_module import MorphoModule


class Erosion(MorphoModule):
    """Learnable erosion layer, (x (-) w)[i, j] = min{x[i+m, j+n] - w[m, n]}; same constructor as the
    reference `morphocore.nn.Erosion` (morphocore/nn/erosion.py:86-101). See
    `morphocore_b200.functional.erosion` for the arguments."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: tuple,
                 channel_merge_mode: str = "sum", padding_mode: str = "replicate",
                 dtype: torch.dtype = torch.float32, save_indices: bool = True,
                 weight_dropout: float = 0.0, padding_value: float = 0.0, noise_scale: float = 0.0):
        if type(kernel_size) is int:
            kernel_size = (kernel_size, kernel_size)
        self.save_indices = save_indices
        self.weight_dropout = weight_dropout
        self.noise_scale = noise_scale
        super().__init__(in_channels, out_channels, kernel_size, channel_merge_mode, padding_mode, dtype=dtype,
                         padding_value=padding_value)

    def forward(self, x):
        return erosion(x, self.weight, self.channel_merge_mode, self.padding_mode,
                        self.save_indices, self.weight_dropout, self.training,
                        self.padding_value, self.noise_scale)

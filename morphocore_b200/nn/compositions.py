"""Composite layers built from Dilation and Erosion, same constructors as the reference
(morphocore/nn/opening.py:104-180, closing.py, sigma_layer.py:91-104)."""
import torch
import torch.nn as nn

from morphocore_b200.functional import sigma_layer
from .alpha_module import AlphaModule
from .dilation import Dilation
from .erosion import Erosion


def _stage_arguments(in_channels, out_channels, kernel_size, channel_merge_mode, share_weights):
    if type(kernel_size) is int:
        kernel_size = (kernel_size, kernel_size)
    # One structuring element for both stages makes the layer an algebraic opening / closing (idempotent,
    # anti-extensive / extensive); that only makes sense channel by channel.
    if share_weights:
        if in_channels != out_channels:
            raise ValueError(f"share_weights=True needs in_channels == out_channels, got {in_channels} and {out_channels}. "
                             "Pass share_weights=False for two independent structuring elements.")
        if channel_merge_mode not in (None, 'identity'):
            raise ValueError(f"share_weights=True forces channel_merge_mode='identity', got '{channel_merge_mode}'. "
                             "Pass share_weights=False to merge channels instead.")
        channel_merge_mode = 'identity'
    elif channel_merge_mode is None:
        channel_merge_mode = 'sum'
    return kernel_size, channel_merge_mode


class _TwoStage(nn.Module):
    first_is_erosion = True

    def __init__(self, in_channels: int, out_channels: int, kernel_size, channel_merge_mode: str = None,
                 padding_mode: str = "replicate", dtype: torch.dtype = torch.float32, save_indices: bool = True,
                 padding_value: float = 0.0, share_weights: bool = True, weight_dropout: float = 0.0, noise_scale: float = 0.0):
        super().__init__()
        kernel_size, channel_merge_mode = _stage_arguments(in_channels, out_channels, kernel_size, channel_merge_mode, share_weights)
        self.share_weights = share_weights
        common = dict(kernel_size=kernel_size, padding_mode=padding_mode, padding_value=padding_value, weight_dropout=weight_dropout,
                      noise_scale=noise_scale, dtype=dtype, save_indices=save_indices)
        first, second = (Erosion, Dilation) if self.first_is_erosion else (Dilation, Erosion)
        stage1 = first(in_channels=in_channels, out_channels=out_channels, channel_merge_mode=channel_merge_mode, **common)
        stage2 = second(in_channels=out_channels, out_channels=out_channels, channel_merge_mode='identity', **common)
        self.erosion, self.dilation = (stage1, stage2) if self.first_is_erosion else (stage2, stage1)
        if share_weights:
            stage2.weight = stage1.weight  # one nn.Parameter behind both stages

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.first_is_erosion:
            return self.dilation(self.erosion(x))
        return self.erosion(self.dilation(x))


class Opening(_TwoStage):
    """Erosion followed by a per-channel dilation."""
    first_is_erosion = True


class Closing(_TwoStage):
    """Dilation followed by a per-channel erosion."""
    first_is_erosion = False


class SigmaLayer(AlphaModule):
    """Learnable blend sigmoid(alpha) * dilation + (1 - sigmoid(alpha)) * erosion with one structuring element."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: tuple, channel_merge_mode: str = "sum",
                 padding_mode: str = "replicate", init_alpha: float = 0.0, dtype: torch.dtype = torch.float32,
                 save_indices: bool = True, padding_value: float = 0.0, weight_dropout: float = 0.0, noise_scale: float = 0.0):
        if type(kernel_size) is int:
            kernel_size = (kernel_size, kernel_size)
        super().__init__(in_channels, out_channels, kernel_size, channel_merge_mode, init_alpha, dtype=dtype)
        self.save_indices = save_indices
        self.padding_mode = padding_mode
        self.padding_value = padding_value
        self.weight_dropout = weight_dropout
        self.noise_scale = noise_scale

    def forward(self, x):
        return sigma_layer(x, self.weight, self.alpha, self.channel_merge_mode, padding_mode=self.padding_mode,
                           save_indices=self.save_indices, padding_value=self.padding_value,
                           weight_dropout=self.weight_dropout, training=self.training, noise_scale=self.noise_scale)
